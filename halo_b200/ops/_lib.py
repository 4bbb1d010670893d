"""ctypes binding to the in-tree sm_100a kernel library.

``lib()`` returns the loaded library or raises: on a machine with a GPU the CUDA kernels are the
only implementation of the hot ops, so a missing library is an error there, never a silent
fallback to eager PyTorch. CPU-only processes (unit tests, gloo ranks) never call ``lib()``; the
op wrappers route CPU tensors to their PyTorch reference implementations instead.
"""

from __future__ import annotations

import ctypes
import threading
from pathlib import Path

import torch

_LIB = None
_LOCK = threading.Lock()
LIB_PATH = Path(__file__).resolve().parent.parent / "lib" / "libhalo_b200.so"

c_void_p = ctypes.c_void_p
c_int = ctypes.c_int
c_ll = ctypes.c_longlong
c_float = ctypes.c_float


class KernelError(RuntimeError):
    """A kernel entry point refused its arguments or a launch failed."""


# kernels launched per entry point (entries that only compute sizes on the host launch none)
_KERNELS_PER_CALL = {
    "halo_rmsnorm_bwd": 2, "halo_qknorm_rope_bwd": 2, "halo_attn_bwd": 3, "halo_route_count": 2, "halo_sq_norm": 2,
    "halo_rmsnorm_bwd_blocks": 0, "halo_qknorm_rope_bwd_blocks": 0, "halo_gemm_work_bytes": 0,
    "halo_rmsnorm_supported": 0, "halo_route_blocks": 0, "halo_adam_elems_per_block": 0,
    "halo_adam_q8_elems_per_block": 0, "halo_adam_q8_group": 0, "halo_moe_push_unit_bytes": 0, "halo_moe_tile_bytes": 0, "halo_moe_ctrl_ints": 0,
}
LAUNCHES = {"total": 0}


class _CountingLib:
    """Thin proxy over the CDLL that counts kernel launches, so a benchmark can report how many of
    this library's kernels ran inside its timed region."""

    def __init__(self, cdll):
        self._cdll = cdll
        self._cache = {}

    def __getattr__(self, name):
        fn = self._cache.get(name)
        if fn is None:
            raw = getattr(self._cdll, name)
            n = _KERNELS_PER_CALL.get(name, 1)

            def fn(*args, _raw=raw, _n=n):
                LAUNCHES["total"] += _n
                return _raw(*args)

            self._cache[name] = fn
        return fn


def launch_count() -> int:
    return LAUNCHES["total"]


def lib():
    global _LIB
    if _LIB is not None:
        return _LIB
    with _LOCK:
        if _LIB is None:
            if not LIB_PATH.exists():
                try:
                    from halo_b200.build_ext import build

                    build()
                except Exception as exc:  # pragma: no cover - depends on the toolchain
                    raise KernelError(
                        f"the sm_100a kernel library {LIB_PATH} is missing and could not be built: {exc}"
                    ) from exc
            _LIB = _CountingLib(ctypes.CDLL(str(LIB_PATH)))
    return _LIB


def available() -> bool:
    """True when CUDA kernels can run in this process (a GPU is visible)."""
    return torch.cuda.is_available()


def ptr(t: torch.Tensor | None) -> c_void_p:
    if t is None:
        return c_void_p(0)
    return c_void_p(t.data_ptr())


def stream_ptr(device: torch.device | None = None) -> c_void_p:
    return c_void_p(torch.cuda.current_stream(device).cuda_stream)


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise KernelError(f"{what} failed with code {rc}")


_STATUS: dict[int, torch.Tensor] = {}


def status_word(device: torch.device) -> torch.Tensor:
    """A per-device int32 the kernels write a non-zero code into when a bounded wait gives up."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _STATUS.get(idx)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
        _STATUS[idx] = t
    return t


def read_status(device: torch.device | None = None, reset: bool = True) -> int:
    """Synchronising read of the status word; call between steps, not inside the hot loop."""
    device = device or torch.device("cuda", torch.cuda.current_device())
    t = status_word(device)
    v = int(t.item())
    if v and reset:
        t.zero_()
    return v


def raise_on_status(device: torch.device | None = None) -> None:
    v = read_status(device)
    if v:
        names = {1: "a wait inside a kernel ran out of its time budget", 2: "bad argument",
                 3: "a wait on a peer GPU ran out of its time budget", 4: "index out of bounds"}
        raise KernelError(f"kernel status {v}: {names.get(v, 'unknown')}")


_HOST_LIB = None


def host_lib():
    """The CPU-side library (``libhalo_host.so``: the host optimizer); built on first use if missing."""
    global _HOST_LIB
    if _HOST_LIB is None:
        from halo_b200.build_ext import HOST_LIB_PATH, build_host

        if not HOST_LIB_PATH.exists():
            build_host()
        _HOST_LIB = ctypes.CDLL(str(HOST_LIB_PATH))
        _HOST_LIB.halo_host_adamw_bf16.restype = ctypes.c_int
        _HOST_LIB.halo_host_threads.restype = ctypes.c_int
    return _HOST_LIB
