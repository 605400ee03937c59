"""Benchmarks that ship with the library (run as ``python -m umdk_original_b200.bench.<name>``)."""
