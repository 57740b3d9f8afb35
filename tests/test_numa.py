"""CPU-list parsing and the no-op behaviour of NUMA binding where the topology is unknown."""
from switchml_b200.utils.numa import parse_cpu_list, bind_to_device_numa, device_numa_node


def test_parse_cpu_list():
    assert parse_cpu_list("0-3,8,10-11") == {0, 1, 2, 3, 8, 10, 11}
    assert parse_cpu_list("") == set() and parse_cpu_list(None) == set()
    assert parse_cpu_list("5") == {5}


def test_binding_without_a_gpu_changes_nothing():
    import os
    before = os.sched_getaffinity(0)
    assert device_numa_node(0) is None or isinstance(device_numa_node(0), int)
    bind_to_device_numa(0)
    assert os.sched_getaffinity(0) <= before
