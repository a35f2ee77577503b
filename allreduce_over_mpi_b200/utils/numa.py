"""Host-memory placement next to a GPU (read-only use of sysfs, plus this process's own CPU affinity).

A pinned host buffer lands on the NUMA node of the thread that first touches it.  On a two-socket host a buffer
on the far socket makes every host<->device copy cross the socket interconnect, which becomes the limit once
several GPUs copy at the same time.  ``bind_to_gpu_node`` moves the calling process onto the CPUs the kernel lists
as local to the GPU's PCIe root (``/sys/bus/pci/devices/<bdf>/local_cpulist``), so that buffers allocated afterwards
sit on the GPU's side.  Nothing outside this process is changed; where sysfs does not say, nothing happens.
"""
from __future__ import annotations

import os


def _parse_cpulist(text: str) -> set[int]:
    cpus: set[int] = set()
    for part in text.strip().split(","):
        if not part:
            continue
        lo, _, hi = part.partition("-")
        cpus.update(range(int(lo), int(hi or lo) + 1))
    return cpus


def gpu_local_cpus(device_index: int) -> tuple[set[int], int | None]:
    """CPUs local to the GPU and its NUMA node, or (empty set, None) when the system does not tell."""
    try:
        import torch
        p = torch.cuda.get_device_properties(device_index)
        bdf = f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
        base = f"/sys/bus/pci/devices/{bdf}"
        cpus = _parse_cpulist(open(f"{base}/local_cpulist").read())
        node = int(open(f"{base}/numa_node").read().strip())
        return cpus, (node if node >= 0 else None)
    except Exception:  # noqa: BLE001 - no sysfs, no such attribute, not a PCI device: no information
        return set(), None


def bind_to_gpu_node(device_index: int) -> dict | None:
    """Restrict this process to the CPUs local to the GPU (those it is allowed to use anyway).  Returns what was done,
    or None when there was nothing to do (no information, or already there)."""
    cpus, node = gpu_local_cpus(device_index)
    try:
        allowed = os.sched_getaffinity(0)
    except AttributeError:
        return None
    target = cpus & allowed
    if not target or target == allowed:
        return None
    os.sched_setaffinity(0, target)
    return {"numa_node": node, "cpus": len(target), "of_allowed": len(allowed)}
