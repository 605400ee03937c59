"""Comparison layer only: NCCL all_to_all_single + cuBLAS expert GEMMs.  Nothing in the product
package imports this directory."""
