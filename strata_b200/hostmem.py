"""Host-side placement for the staging buffers of host-buffer calls.

A GPU's PCIe root port hangs off one CPU socket.  Pinned host memory that lives on the other socket's NUMA node
makes every host<->device copy cross the inter-socket link, which eight ranks copying at once saturate.  Linux
places pages on the node of the CPU that first touches them, so a rank that restricts itself to the CPUs of its
GPU's node BEFORE it allocates its pinned buffers gets local staging memory without any NUMA library.

The topology comes from sysfs, like the reference's host topology reader (src/platform/numa_topology.cpp:19-45 parses
the same `cpulist` format; its placement calls serve host-resident weights, include/strata/numa_topology.hpp:53-60).
Everything here is best effort: a container without the sysfs entries, with one node, or with a CPU set that has no
CPU on the GPU's node is left as it is.
"""
import os


def parse_cpu_list(text):
    """'0-13,28-41' -> [0..13, 28..41]; malformed items are skipped."""
    cpus = []
    for item in text.strip().split(","):
        item = item.strip()
        if not item:
            continue
        lo, dash, hi = item.partition("-")
        try:
            first = int(lo)
            last = int(hi) if dash else first
        except ValueError:
            continue
        cpus.extend(range(first, last + 1))
    return cpus


def gpu_numa_node(pci_bus_id, sysfs="/sys"):
    """NUMA node of the PCI function 'dddd:bb:dd.f' (-1 or None when the kernel does not say)."""
    path = os.path.join(sysfs, "bus", "pci", "devices", pci_bus_id.lower(), "numa_node")
    try:
        with open(path) as f:
            return int(f.read().strip())
    except (OSError, ValueError):
        return None


def node_cpus(node, sysfs="/sys"):
    try:
        with open(os.path.join(sysfs, "devices", "system", "node", "node%d" % node, "cpulist")) as f:
            return parse_cpu_list(f.read())
    except OSError:
        return []


def bind_near_gpu(device_index, sysfs="/sys", allowed=None, apply=True):
    """Restrict the calling process to the CPUs of the NUMA node the GPU is attached to.

    Call before allocating pinned staging buffers.  Returns a record for logs:
    {"node": n or None, "cpus": count, "bound": bool, "why": reason when not bound}.
    `allowed` (default: the current affinity mask) and `apply=False` exist for tests.
    """
    rec = {"node": None, "cpus": 0, "bound": False}
    try:
        import torch
        p = torch.cuda.get_device_properties(device_index)
        bus = "%04x:%02x:%02x.0" % (p.pci_domain_id, p.pci_bus_id, p.pci_device_id)
    except Exception as e:    # no CUDA, or a torch without the PCI fields
        rec["why"] = "no PCI address: %s" % type(e).__name__
        return rec
    return bind_to_node_of(bus, sysfs=sysfs, allowed=allowed, apply=apply, rec=rec)


def bind_to_node_of(pci_bus_id, sysfs="/sys", allowed=None, apply=True, rec=None):
    rec = rec if rec is not None else {"node": None, "cpus": 0, "bound": False}
    node = gpu_numa_node(pci_bus_id, sysfs)
    rec["node"] = node
    if node is None or node < 0:
        rec["why"] = "the kernel reports no node for the device"
        return rec
    if allowed is None:
        allowed = os.sched_getaffinity(0)
    cpus = sorted(set(node_cpus(node, sysfs)) & set(allowed))
    rec["cpus"] = len(cpus)
    if not cpus:
        rec["why"] = "no allowed CPU on the device's node"
        return rec
    if len(cpus) == len(set(allowed)):
        rec["why"] = "already confined to that node"
        return rec
    if apply:
        try:
            os.sched_setaffinity(0, cpus)
        except OSError as e:
            rec["why"] = "sched_setaffinity: %s" % e
            return rec
    rec["bound"] = True
    return rec
