"""Facts about the machine: GPU generation, peak rates (nominal and measured on this box), host
memory, CPU quota and free disk (the role of halo/hardware.py:20-245).

The roofline denominators are the *measured* copy bandwidth and bf16 GEMM rate of the box when a
``MEASURED_PEAKS.json`` sits at the repository root; the nominal table is context only.
"""

from __future__ import annotations

import json
import os
import shutil
from dataclasses import dataclass
from pathlib import Path

# dense peaks per GPU, FLOP/s (the doubled marketing figures are with 2:4 sparsity)
GPU_PEAK_FLOPS = {
    "B200": {"bf16": 2.25e15, "fp16": 2.25e15, "fp8": 4.5e15, "fp4": 9.0e15, "tf32": 1.1e15},
    "B300": {"bf16": 2.25e15, "fp16": 2.25e15, "fp8": 4.5e15, "fp4": 13.5e15, "tf32": 1.1e15},
    "H100": {"bf16": 0.989e15, "fp16": 0.989e15, "fp8": 1.979e15, "tf32": 0.494e15},
    "H200": {"bf16": 0.989e15, "fp16": 0.989e15, "fp8": 1.979e15, "tf32": 0.494e15},
    "A100": {"bf16": 0.312e15, "fp16": 0.312e15, "tf32": 0.156e15},
}
B200 = {"sms": 148, "hbm_bytes": 180e9, "hbm_gbs_nominal": 7700.0, "l2_bytes": 126e6, "smem_per_cta": 227 * 1024,
        "tmem_columns": 512, "nvlink_gbs_per_direction": 900.0, "nvlink_gbs_measured_peer_copy": 770.0,
        "allreduce_busbw_gbs_measured": 725.0}

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


@dataclass(frozen=True)
class MeasuredPeaks:
    hbm_gbs: float
    bf16_tflops: float
    bf16_tflops_sustained: float
    source: str  # "measured" or "fallback"

    def label(self) -> str:
        return "of measured" if self.source == "measured" else "of fallback"


def measured_peaks(root: str | os.PathLike | None = None) -> MeasuredPeaks:
    root = Path(root) if root else Path(__file__).resolve().parent.parent
    path = root / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            d = json.loads(path.read_text())
            return MeasuredPeaks(float(d["hbm_gbs"]), float(d["bf16_tflops"]),
                                 float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "measured")
        except (ValueError, KeyError):
            pass
    return MeasuredPeaks(FALLBACK_PEAKS["hbm_gbs"], FALLBACK_PEAKS["bf16_tflops"],
                         FALLBACK_PEAKS["bf16_tflops_sustained"], "fallback")


def cuda_capability() -> tuple[int, int] | None:
    try:
        import torch

        if torch.cuda.is_available():
            return torch.cuda.get_device_capability()
    except Exception:  # pragma: no cover
        pass
    return None


def is_blackwell_gpu() -> bool:
    cap = cuda_capability()
    return cap is not None and cap[0] >= 10


def is_hopper_gpu() -> bool:
    cap = cuda_capability()
    return cap is not None and cap[0] == 9


def supports_tcgen05() -> bool:
    """The kernels of this package are built for sm_100a only."""
    cap = cuda_capability()
    return cap is not None and cap[0] == 10


def gpu_sku(name: str | None = None) -> str | None:
    if name is None:
        try:
            import torch

            name = torch.cuda.get_device_name() if torch.cuda.is_available() else None
        except Exception:  # pragma: no cover
            name = None
    if not name:
        return None
    for sku in GPU_PEAK_FLOPS:
        if sku in name.upper():
            return sku
    return None


def peak_flops(dtype: str = "bf16", name: str | None = None) -> float | None:
    sku = gpu_sku(name)
    return GPU_PEAK_FLOPS.get(sku, {}).get(dtype) if sku else None


def host_memory_bytes() -> int:
    """Physical memory visible to this process, honouring a cgroup limit."""
    total = os.sysconf("SC_PAGE_SIZE") * os.sysconf("SC_PHYS_PAGES")
    for p in ("/sys/fs/cgroup/memory.max", "/sys/fs/cgroup/memory/memory.limit_in_bytes"):
        try:
            raw = Path(p).read_text().strip()
            if raw.isdigit():
                total = min(total, int(raw))
        except OSError:
            continue
    return total


def cpu_quota() -> float:
    """CPUs this process may use (cgroup quota or the affinity mask)."""
    try:
        raw = Path("/sys/fs/cgroup/cpu.max").read_text().split()
        if raw and raw[0] != "max":
            return max(1.0, int(raw[0]) / int(raw[1]))
    except (OSError, ValueError, IndexError):
        pass
    try:
        return float(len(os.sched_getaffinity(0)))
    except AttributeError:  # pragma: no cover
        return float(os.cpu_count() or 1)


def free_disk_bytes(path: str) -> int:
    probe = Path(path)
    while not probe.exists() and probe != probe.parent:
        probe = probe.parent
    return shutil.disk_usage(probe).free
