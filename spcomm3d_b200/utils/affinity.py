"""Host placement of a rank next to its GPU.

The pinned staging buffers of a rank should live in the memory of the NUMA
node its GPU hangs off: a copy from the other socket crosses the inter-socket
link and shares it with every other rank that does the same.  Pinned pages
are placed on the node of the allocating thread, so it is enough to restrict
the process to the CPUs of the GPU's node before the first pinned allocation.
The node and its CPUs are read from sysfs; nothing is changed on the GPU.

The reference leaves placement to the MPI launcher (one rank per core, bound by
`mpirun`/`srun` options outside the code base).
"""
from __future__ import annotations

import os


def parse_cpulist(text: str) -> set[int]:
    """"0-3,8,10-11" -> {0, 1, 2, 3, 8, 10, 11}."""
    cpus: set[int] = set()
    for part in text.strip().split(","):
        if not part:
            continue
        lo, _, hi = part.partition("-")
        cpus.update(range(int(lo), int(hi or lo) + 1))
    return cpus


def pci_address(device_index: int) -> str | None:
    """"dddd:bb:dd.0" of a visible CUDA device, or None if torch does not expose it."""
    import torch
    try:
        props = torch.cuda.get_device_properties(device_index)
    except (RuntimeError, AssertionError):
        return None
    bus, dev = getattr(props, "pci_bus_id", None), getattr(props, "pci_device_id", None)
    if bus is None or dev is None:
        return None
    return f"{getattr(props, 'pci_domain_id', 0):04x}:{bus:02x}:{dev:02x}.0"


def numa_node_of(pci: str, sysfs: str = "/sys") -> int | None:
    try:
        with open(os.path.join(sysfs, "bus/pci/devices", pci, "numa_node")) as f:
            node = int(f.read().strip())
    except (OSError, ValueError):
        return None
    return node if node >= 0 else None


def node_cpus(node: int, sysfs: str = "/sys") -> set[int]:
    try:
        with open(os.path.join(sysfs, f"devices/system/node/node{node}/cpulist")) as f:
            return parse_cpulist(f.read())
    except (OSError, ValueError):
        return set()


def bind_near(pci: str | None, sysfs: str = "/sys", slot: int = 0, nslots: int = 1, apply: bool = True) -> dict:
    """Restricts this process to the CPUs of the NUMA node of the PCI device `pci` that it is already allowed
    to use; with nslots > 1 ranks sharing a node, rank `slot` takes the slot-th share of them (a private core
    set).  Returns {"node", "cpus"}; node None = nothing known, nothing changed."""
    info = {"node": None, "cpus": 0}
    if pci is None or not hasattr(os, "sched_getaffinity"):
        return info
    node = numa_node_of(pci, sysfs)
    if node is None:
        return info
    allowed = sorted(node_cpus(node, sysfs) & os.sched_getaffinity(0))
    if not allowed:
        return info
    if nslots > 1 and len(allowed) >= nslots:
        per = len(allowed) // nslots
        allowed = allowed[slot * per:(slot + 1) * per]
    if apply:
        try:
            os.sched_setaffinity(0, allowed)
        except OSError:
            return info
    info["node"], info["cpus"] = node, len(allowed)
    return info


def bind_near_gpu(device_index: int, local_rank: int = 0, local_world: int = 1) -> dict:
    """`bind_near` for a CUDA device; SP3_NUMA_BIND=0 switches it off.  Ranks of one node that share a NUMA
    node split its CPUs: the share is chosen from the local rank, assuming the ranks are spread evenly over
    the two halves of the GPUs (rank r of W -> share r mod (W / nodes))."""
    if os.environ.get("SP3_NUMA_BIND", "1") != "1":
        return {"node": None, "cpus": 0}
    try:
        n_nodes = len([d for d in os.listdir("/sys/devices/system/node") if d.startswith("node") and d[4:].isdigit()])
    except OSError:
        n_nodes = 1
    per_node = max(1, -(-local_world // max(n_nodes, 1)))
    return bind_near(pci_address(device_index), slot=local_rank % per_node, nslots=per_node)
