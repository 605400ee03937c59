"""Host-side helpers: CPU-list parsing and NUMA binding that never raises."""
from umdk_original_b200.utils import host


def test_parse_cpulist():
    assert host._parse_cpulist("0-3,8,10-11\n") == {0, 1, 2, 3, 8, 10, 11}
    assert host._parse_cpulist("") == set()


def test_bind_without_gpu_is_a_no_op():
    # no CUDA device here: the lookup fails and the affinity stays as it is
    import os
    before = os.sched_getaffinity(0) if hasattr(os, "sched_getaffinity") else None
    assert host.bind_to_gpu_numa_node(0) in (None, 0, 1, 2, 3)
    if before is not None and host.gpu_numa_node(0) is None:
        assert os.sched_getaffinity(0) == before


def test_nvtx_range_is_a_no_op_without_a_gpu_or_when_disabled():
    from umdk_original_b200.utils import nvtx
    was = nvtx.enabled()
    try:
        for on in (False, True):
            nvtx.enable(on)
            with nvtx.nvtx_range("probe"):
                pass
    finally:
        nvtx.enable(was)
