"""Keeps a rank's host memory next to its GPU.

Pinned host buffers are placed on the NUMA node of the thread that first touches them.  Ranks started
by ``torchrun`` run wherever the scheduler puts them, so on a two-socket host half of the ranks feed
their GPU across the socket interconnect, and with several GPUs copying at once that interconnect, not
PCIe, bounds the aggregate host-to-device rate.  :func:`bind_to_gpu_node` restricts the calling process
to the CPUs of the NUMA node that the GPU's PCIe root port hangs off (read from sysfs), before any
pinned allocation is made.

Nothing is changed when the information is missing (``numa_node`` of -1, a container without the
sysfs files), when the node's CPUs are outside the process's allowed set, or when
``TILECCL_NO_NUMA_BIND=1`` is set; the function never raises.  Only the calling process's own CPU
affinity is touched, no setting of the GPU or of the machine.

The reference binds nothing (its transfers are device to device); this serves the host-to-device leg
of the end-to-end benchmark.
"""
from __future__ import annotations

import os


def parse_cpulist(text: str) -> set[int]:
    """``"0-3,8,10-11"`` -> {0, 1, 2, 3, 8, 10, 11}."""
    cpus: set[int] = set()
    for part in text.strip().split(","):
        part = part.strip()
        if not part:
            continue
        if "-" in part:
            lo, hi = part.split("-", 1)
            cpus.update(range(int(lo), int(hi) + 1))
        else:
            cpus.add(int(part))
    return cpus


def gpu_numa_node(pci_bus_id: str, sysfs: str = "/sys") -> int:
    """NUMA node of the PCI device ``domain:bus:device.function`` (-1 if unknown)."""
    bdf = pci_bus_id.strip().lower()
    if bdf.count(":") == 2 and len(bdf.split(":")[0]) == 8:      # NVML pads the domain to 8 hex digits, sysfs uses 4
        bdf = bdf[4:]
    try:
        with open(os.path.join(sysfs, "bus", "pci", "devices", bdf, "numa_node")) as f:
            return int(f.read().strip())
    except (OSError, ValueError):
        return -1


def node_cpus(node: int, sysfs: str = "/sys") -> set[int]:
    try:
        with open(os.path.join(sysfs, "devices", "system", "node", f"node{node}", "cpulist")) as f:
            return parse_cpulist(f.read())
    except (OSError, ValueError):
        return set()


def bind_to_gpu_node(device: int | None = None, sysfs: str = "/sys", pci_bus_id: str | None = None) -> dict:
    """Restricts this process to the CPUs of the GPU's NUMA node.  Returns what was found and done:
    ``{"node": n, "cpus": k, "bound": bool, "why": "..."}``."""
    info = {"node": -1, "cpus": 0, "bound": False, "why": ""}
    try:
        if os.environ.get("TILECCL_NO_NUMA_BIND") == "1":
            info["why"] = "disabled by TILECCL_NO_NUMA_BIND"
            return info
        if pci_bus_id is None:
            import torch
            dev = torch.cuda.current_device() if device is None else device
            props = torch.cuda.get_device_properties(dev)
            pci_bus_id = f"{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
        node = gpu_numa_node(pci_bus_id, sysfs)
        info["node"] = node
        if node < 0:
            info["why"] = "the GPU's NUMA node is not reported"
            return info
        want = node_cpus(node, sysfs)
        allowed = os.sched_getaffinity(0)
        use = want & allowed
        info["cpus"] = len(use)
        if not use:
            info["why"] = "the node's CPUs are outside this process's allowed set"
            return info
        if use == allowed:
            info["why"] = "already confined to the node"
            info["bound"] = True
            return info
        os.sched_setaffinity(0, use)
        info["bound"] = True
        info["why"] = "affinity set"
    except Exception as e:  # noqa: BLE001  (a convenience: never in the way of the run)
        info["why"] = f"{type(e).__name__}: {e}"
    return info
