"""Keeping a worker process next to its GPU.

Pinned host buffers should live on the NUMA node the GPU hangs off, otherwise every
host<->device copy crosses the socket interconnect and the workers of one box queue up on
one memory controller. The reference pins its RDMA worker threads to cores on the NIC's NUMA
node for the same reason (backends/rdma/rdma_utils.h:135-204: GetDeviceNuma, GetCoresNuma,
BindToCore). ``bind_to_device_numa`` restricts the calling process to the CPUs of the GPU's
node; memory it allocates (and pins) afterwards is placed there by first touch.
"""
import os


def _read(path):
    try:
        with open(path) as f:
            return f.read().strip()
    except OSError:
        return None


def parse_cpu_list(text):
    """'0-3,8,10-11' -> {0,1,2,3,8,10,11}"""
    cpus = set()
    for part in (text or "").split(","):
        part = part.strip()
        if not part:
            continue
        if "-" in part:
            a, b = part.split("-", 1)
            cpus.update(range(int(a), int(b) + 1))
        else:
            cpus.add(int(part))
    return cpus


def device_numa_node(device_index):
    """NUMA node of a CUDA device, or None when the platform does not say."""
    try:
        import torch
        bus = torch.cuda.get_device_properties(device_index).pci_bus_id
        dom = torch.cuda.get_device_properties(device_index).pci_domain_id
        dev = torch.cuda.get_device_properties(device_index).pci_device_id
    except Exception:
        return None
    name = "%04x:%02x:%02x.0" % (dom, bus, dev)
    node = _read("/sys/bus/pci/devices/%s/numa_node" % name)
    if node is None or int(node) < 0:
        return None
    return int(node)


def bind_to_device_numa(device_index):
    """Restrict this process to the CPUs of the device's NUMA node. Returns the node, or
    None if nothing was changed (unknown topology, single node, or not permitted)."""
    node = device_numa_node(device_index)
    if node is None:
        return None
    cpus = parse_cpu_list(_read("/sys/devices/system/node/node%d/cpulist" % node))
    try:
        allowed = os.sched_getaffinity(0)
        target = cpus & allowed
        if not target or target == allowed:
            return None
        os.sched_setaffinity(0, target)
    except (OSError, AttributeError):
        return None
    return node
