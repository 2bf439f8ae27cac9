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


def nvml_cpu_affinity(device_index: int, nvml=None) -> set[int]:
    """CPUs that the driver names as close to a visible CUDA device (a read-only NVML query), or an empty set.
    The device is found by its UUID, so a remapped CUDA_VISIBLE_DEVICES does not matter."""
    try:
        import torch
        if nvml is None:
            import pynvml as nvml
            nvml.nvmlInit()
        uuid = str(torch.cuda.get_device_properties(device_index).uuid)
        handle = nvml.nvmlDeviceGetHandleByUUID(uuid if uuid.startswith("GPU-") else "GPU-" + uuid)
        words = nvml.nvmlDeviceGetCpuAffinity(handle, ((os.cpu_count() or 64) + 63) // 64)
    except Exception:   # no driver, no NVML, an old torch without uuid: placement is best effort
        return set()
    return {64 * w + b for w, word in enumerate(words) for b in range(64) if int(word) >> b & 1}


def bind_to(cpus: set[int], slot: int = 0, nslots: int = 1, apply: bool = True) -> int:
    """Restricts this process to the slot-th of nslots shares of `cpus` (those it may already use);
    returns the number of CPUs it ends up with, 0 = nothing changed."""
    if not cpus or not hasattr(os, "sched_getaffinity"):
        return 0
    allowed = sorted(cpus & os.sched_getaffinity(0))
    if nslots > 1 and len(allowed) >= nslots:
        per = len(allowed) // nslots
        allowed = allowed[slot * per:(slot + 1) * per]
    if not allowed:
        return 0
    if apply:
        try:
            os.sched_setaffinity(0, allowed)
        except OSError:
            return 0
    return len(allowed)


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
    slot = local_rank % per_node
    info = bind_near(pci_address(device_index), slot=slot, nslots=per_node)
    if info["node"] is None:
        # sysfs names no node (a container without it): ask the driver which CPUs are close to the GPU; a set
        # that covers every CPU of the machine says nothing and is left alone
        cpus = nvml_cpu_affinity(device_index)
        if cpus and len(cpus) < (os.cpu_count() or 0):
            info = {"node": "nvml", "cpus": bind_to(cpus, slot, per_node)}
    return info
