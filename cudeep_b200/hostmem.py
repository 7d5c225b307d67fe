"""Host memory next to a GPU.

The host-buffer entry points (`cudeep_b200_matmul_host_f32` and friends) are bound by the host link:
an 8192^3 product moves 805 MB over PCIe for 1.4 ms of tensor-core time.  On a two-socket host the
link of a GPU hangs off one socket, and pinned buffers whose pages live on the other socket cross the
socket interconnect on every copy (the same call has been measured at 11 ms on some machines of one
pool and at 16 and 26 ms on others).  Linux places the pages of a new allocation on the NUMA node of the thread that first touches them,
so allocating the pinned buffers from a thread that runs on the GPU's node is enough.

`near_gpu(index)` does that for the calling thread: it narrows the thread's CPU affinity to the CPUs
of the GPU's NUMA node for the duration of a `with` block and restores it afterwards.  It reads
sysfs only; it changes nothing about the GPU.  Where sysfs does not say (no NUMA, a container
without /sys, an unknown PCI address) it does nothing and says so in what it returns.
"""
from __future__ import annotations

import contextlib
import os
from pathlib import Path

SYSFS = Path("/sys")


def parse_cpulist(text: str) -> set[int]:
    """'0-3,8,10-11' -> {0, 1, 2, 3, 8, 10, 11} (the format of sysfs cpulist files)."""
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


def pci_address(index: int) -> str | None:
    """'0000:1b:00.0' for CUDA device `index` of this process, through NVML (read-only); None if
    NVML is not there.  NVML counts all GPUs of the machine, CUDA only the visible ones, so the
    device is looked up by the UUID CUDA reports when torch is importable."""
    try:
        import pynvml
        pynvml.nvmlInit()
        handle = None
        try:
            import torch
            uuid = str(torch.cuda.get_device_properties(index).uuid)
            want = uuid if uuid.startswith("GPU-") else "GPU-" + uuid
            handle = pynvml.nvmlDeviceGetHandleByUUID(want.encode())
        except Exception:
            handle = pynvml.nvmlDeviceGetHandleByIndex(index)
        bus = pynvml.nvmlDeviceGetPciInfo(handle).busId
        bus = bus.decode() if isinstance(bus, bytes) else bus
        # NVML prints an 8-digit domain, sysfs a 4-digit one.
        domain, rest = bus.split(":", 1)
        return f"{int(domain, 16):04x}:{rest}".lower()
    except Exception:
        return None


def numa_node_of(pci: str, sysfs: Path = SYSFS) -> int | None:
    """NUMA node of a PCI device, or None when sysfs has no answer (-1 means 'no NUMA')."""
    try:
        node = int((sysfs / "bus" / "pci" / "devices" / pci / "numa_node").read_text().strip())
    except (OSError, ValueError):
        return None
    return node if node >= 0 else None


def cpus_of_node(node: int, sysfs: Path = SYSFS) -> set[int]:
    try:
        return parse_cpulist((sysfs / "devices" / "system" / "node" / f"node{node}" / "cpulist").read_text())
    except (OSError, ValueError):
        return set()


@contextlib.contextmanager
def near_gpu(index: int = 0, sysfs: Path = SYSFS, pci: str | None = None):
    """Runs the block with the calling thread confined to the CPUs of the GPU's NUMA node.

    Yields a dict: {"pci": ..., "numa_node": ..., "cpus": <how many CPUs the thread may use inside
    the block>, "bound": <whether the affinity was narrowed>}."""
    info = {"pci": pci or pci_address(index), "numa_node": None, "cpus": None, "bound": False}
    saved = None
    try:
        if info["pci"] is not None and hasattr(os, "sched_getaffinity"):
            node = numa_node_of(info["pci"], sysfs)
            info["numa_node"] = node
            if node is not None:
                allowed = os.sched_getaffinity(0)
                local = cpus_of_node(node, sysfs) & allowed
                if local and local != allowed:
                    saved = allowed
                    os.sched_setaffinity(0, local)
                    info["bound"] = True
                info["cpus"] = len(local) if local else len(allowed)
        yield info
    finally:
        if saved is not None:
            os.sched_setaffinity(0, saved)
