"""Pin a worker process to the CPUs next to its GPU.

The reference binds every learner / engine actor to a NUMA node with libnuma, choosing the node from the local rank
(``open_instruct/utils.py:1594-1617``: ``node = local_rank // (8 // nodes)``).  Here the node is read from the GPU's PCI
device in sysfs (``/sys/bus/pci/devices/<bus id>/numa_node``) and the binding is done by the host runtime
(``b200_numa_bind``: ``sched_setaffinity`` to the node's ``cpulist``; memory then follows by first touch); the rank formula
is the fallback when sysfs does not say.  ``B200_NUMA_BIND=0`` switches it off.  Never fatal: a worker that cannot be pinned
runs unpinned.
"""

from __future__ import annotations

import ctypes
import logging
import os
import re

logger = logging.getLogger(__name__)


def numa_node_count(sysfs: str = "/sys") -> int:
    base = os.path.join(sysfs, "devices/system/node")
    try:
        return sum(1 for n in os.listdir(base) if re.fullmatch(r"node\d+", n))
    except OSError:
        return 0


def pci_numa_node(pci_bus_id: str, sysfs: str = "/sys") -> int | None:
    """NUMA node of a PCI device (``0000:1b:00.0``), or None when the platform reports none (-1) or the file is missing."""
    for name in (pci_bus_id.lower(), pci_bus_id.lower()[-12:]):   # the driver prints an 8-digit domain, sysfs a 4-digit one
        try:
            node = int(open(os.path.join(sysfs, "bus/pci/devices", name, "numa_node")).read().strip())
            return node if node >= 0 else None
        except (OSError, ValueError):
            continue
    return None


def node_for_gpu(device_index: int, pci_bus_id: str | None = None, gpus_per_host: int = 8, sysfs: str = "/sys") -> int | None:
    nodes = numa_node_count(sysfs)
    if nodes <= 1:
        return None if nodes == 0 else 0
    if pci_bus_id:
        node = pci_numa_node(pci_bus_id, sysfs)
        if node is not None:
            return node
    per_node = max(1, gpus_per_host // nodes)
    return min(nodes - 1, device_index // per_node)


def bind_to_gpu(device) -> int | None:
    """Bind the calling process to the NUMA node of CUDA ``device``.  Returns the node, or None when nothing was done."""
    if os.environ.get("B200_NUMA_BIND", "1") != "1":
        return None
    try:
        import torch

        dev = torch.device(device)
        if dev.type != "cuda" or not torch.cuda.is_available():
            return None
        idx = dev.index if dev.index is not None else torch.cuda.current_device()
        props = torch.cuda.get_device_properties(idx)
        bus = None
        if hasattr(props, "pci_bus_id"):
            bus = f"{getattr(props, 'pci_domain_id', 0):04x}:{props.pci_bus_id:02x}:{getattr(props, 'pci_device_id', 0):02x}.0"
        node = node_for_gpu(idx, bus, gpus_per_host=max(1, torch.cuda.device_count()))
        if node is None:
            return None
        return node if bind_to_node(node) > 0 else None
    except Exception as e:  # noqa: BLE001 - pinning is an optimisation
        logger.warning("NUMA binding skipped: %r", e)
        return None


def bind_to_node(node: int) -> int:
    """CPUs in the new affinity mask (0: unknown node, -1: the kernel refused)."""
    from ..ops import lib

    host = lib.load_host()
    host.b200_numa_bind.argtypes = [ctypes.c_int]
    host.b200_numa_bind.restype = ctypes.c_int
    n = int(host.b200_numa_bind(int(node)))
    if n > 0:
        logger.info("bound to NUMA node %d (%d CPUs)", node, n)
    return n
