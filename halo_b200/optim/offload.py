"""AdamWBF16 with the moments of the large tensors kept in page-locked host memory.

A model whose weights, gradients and both moments do not fit one GPU (the 30B-A3B shape on a single
B200: 8 bytes per parameter = 244 GB) can still take exact AdamWBF16 steps: the two bf16 moments
of every large tensor live in host memory and stream through a double-buffered device staging area
while the step kernel runs - host->device copies of the next buckets, the update of bucket i and
device->host copies of the previous ones overlap on three streams (four staging slots, so both
DMA directions stay busy). The arithmetic, the rounding noise and the clip / skip
contract are those of :class:`AdamWBF16`; only the placement of the state differs.

The reference has no counterpart: it shards optimizer state over ranks instead
(halo/checkpoint/parallel/optimizer.py) and does not run its large MoE shapes on one GPU.
"""

from __future__ import annotations

import ctypes
import threading
import time

import torch

from halo_b200.ops import _lib

from .adamw_bf16 import AdamWBF16, param_name_hash

HOST_STATE_MIN_NUMEL = 8 * 1024 * 1024  # smaller tensors keep their moments on the device
STAGING_SLOTS = 4  # >= 3 so that the host->device and device->host copies of neighbouring buckets overlap


class _PinGuard:
    """Unregisters a page-locked range when the tensor that owns it goes away (a later allocation may get the
    same pages back from the C allocator, and registering a range twice is an error)."""

    def __init__(self, ptr: int):
        self.ptr = ptr

    def __del__(self):
        try:
            torch.cuda.cudart().cudaHostUnregister(self.ptr)
        except Exception:  # noqa: BLE001 - interpreter shutdown
            pass


def _pinned_zeros(numel: int, dtype: torch.dtype) -> torch.Tensor:
    """Zero-filled host tensor registered with CUDA as page-locked, without the size rounding of
    torch's pinned-memory cache (which would waste up to 2x on multi-hundred-MB tensors). The registered
    range is made of whole pages that belong to this tensor alone: two registrations must never share a page."""
    page = 4096
    nbytes = numel * torch.empty((), dtype=dtype).element_size()
    raw = torch.zeros(nbytes + 2 * page, dtype=torch.uint8)
    off = (-raw.data_ptr()) % page
    t = raw[off:off + nbytes].view(dtype)
    if torch.cuda.is_available():
        span = (nbytes + page - 1) // page * page
        rc = torch.cuda.cudart().cudaHostRegister(raw.data_ptr() + off, max(span, page), 0)
        if int(rc) != 0:
            raise RuntimeError(f"cudaHostRegister failed with {rc} for {span} bytes")
        t._halo_pin = _PinGuard(raw.data_ptr() + off)
    return t


def host_update_rate(n: int = 1 << 25) -> float:
    """Parameters per second of the host-CPU AdamWBF16 on this machine (all cores), from a short run."""
    L = _lib.host_lib()
    t = [torch.zeros(n, dtype=torch.bfloat16) for _ in range(4)]
    u = [ctypes.c_void_p(x.data_ptr()) for x in t]
    best = 0.0
    for _ in range(2):
        t0 = time.perf_counter()
        L.halo_host_adamw_bf16(u[0], u[1], u[2], u[3], ctypes.c_longlong(n), ctypes.c_ulonglong(1), ctypes.c_ulonglong(2),
                               ctypes.c_ulonglong(3), ctypes.c_float(0.9), ctypes.c_float(0.999), ctypes.c_float(1e-3),
                               ctypes.c_float(0.05), ctypes.c_float(1e-8), ctypes.c_float(1.0), ctypes.c_float(1.0),
                               ctypes.c_int(0), ctypes.c_int(0))
        best = max(best, n / (time.perf_counter() - t0))
    return best


# The host update moves 4 bytes per parameter over PCIe (gradient out, weight in) instead of 8 (both moments in and
# out); it pays when the CPU keeps up with the halved transfer: about 27 GB/s per direction with both directions busy.
HOST_COMPUTE_MIN_RATE = 8.4e9


class HostStateAdamWBF16(AdamWBF16):
    def __init__(self, params, *args, host_min_numel: int = HOST_STATE_MIN_NUMEL,
                 device_state_budget_bytes: int = 0, host_compute: bool | str = False, **kwargs):
        """``host_compute``: update the host-resident tensors ON the host CPU (bit-identical C++ kernel; gradient
        goes out, weight comes back) instead of streaming their moments through the device. Off by default: on the
        16-core hosts of the benchmark machines the streamed path is 2.6 times faster (3.2 s against 8.5 s per step
        of the 30B model), although a short CPU probe in isolation suggests otherwise. ``"auto"`` decides from that
        probe and is only sensible on hosts with many more cores."""
        super().__init__(params, *args, **kwargs)
        if host_compute == "auto":
            try:
                self.host_rate = host_update_rate()
            except Exception:  # noqa: BLE001 - no compiler / library on this machine: keep streaming
                self.host_rate = 0.0
            host_compute = self.host_rate >= HOST_COMPUTE_MIN_RATE
        self.host_compute = bool(host_compute)
        self._worker = None
        self._cpu_flags: dict = {}
        self._g_host = None
        self._cpu_streams = None
        self.host_min_numel = host_min_numel
        # moments of large tensors stay on the device while this budget lasts (4 bytes per element)
        self.device_budget = int(device_state_budget_bytes)
        self._staging = None
        self._streams = None
        self._slot_free = None
        self._opt_stream = None
        self.ready_events: dict = {}   # parameter -> event recorded after its streamed update

    def _on_host(self, p) -> bool:
        return p.is_cuda and p.dtype == torch.bfloat16 and p.numel() >= self.host_min_numel

    def _state_for(self, p, group):
        st = self.state[p]
        if not st and self._on_host(p) and self.device_budget >= 4 * p.numel():
            self.device_budget -= 4 * p.numel()
            return super()._state_for(p, group)
        if not st and self._on_host(p):
            st["step"] = 0
            st["exp_avg"] = _pinned_zeros(p.numel(), torch.bfloat16)
            st["exp_avg_sq"] = _pinned_zeros(p.numel(), torch.bfloat16)
            st["host_state"] = True
            return st
        return super()._state_for(p, group)

    def _ensure_staging(self, device, max_numel: int):
        if self._staging is None or self._staging[0][0].numel() < max_numel:
            self._staging = [
                (torch.empty(max_numel, dtype=torch.bfloat16, device=device),
                 torch.empty(max_numel, dtype=torch.bfloat16, device=device))
                for _ in range(STAGING_SLOTS)
            ]
            self._streams = (torch.cuda.Stream(device), torch.cuda.Stream(device))
            self._opt_stream = torch.cuda.Stream(device)
            self._slot_free = [torch.cuda.Event() for _ in range(STAGING_SLOTS)]
            for ev in self._slot_free:
                ev.record(torch.cuda.current_stream(device))

    def _cuda_step(self, gi, items, device, gdtype, b1, b2, step_size, bc2_sqrt, eps, wd_factor, step):
        on_dev = [it for it in items if not it[2].get("host_state")]
        on_host = [it for it in items if it[2].get("host_state")]
        if on_dev:
            super()._cuda_step(gi, on_dev, device, gdtype, b1, b2, step_size, bc2_sqrt, eps, wd_factor, step)
        if not on_host:
            return
        if self.host_compute:
            return self._host_compute_step(on_host, device, b1, b2, step_size, bc2_sqrt, eps, wd_factor, step)
        L = _lib.lib()
        self._ensure_staging(device, max(p.numel() for _, p, _ in on_host))
        h2d, d2h = self._streams
        main = torch.cuda.current_stream(device)
        # The streamed updates run on their own stream, so the next step's forward can start on the
        # layers that are already updated while later layers are still crossing PCIe. Consumers call
        # wait_ready() before they read a parameter.
        compute = self._opt_stream
        compute.wait_stream(main)   # gradients, clip coefficient and skip flag are final
        for i, (name, p, st) in enumerate(on_host):
            slot = i % STAGING_SLOTS
            n = p.numel()
            m_dev, v_dev = self._staging[slot][0][:n], self._staging[slot][1][:n]
            h2d.wait_event(self._slot_free[slot])
            with torch.cuda.stream(h2d):
                m_dev.copy_(st["exp_avg"], non_blocking=True)
                v_dev.copy_(st["exp_avg_sq"], non_blocking=True)
                ev_in = torch.cuda.Event()
                ev_in.record(h2d)
            compute.wait_event(ev_in)
            g = p.grad.contiguous()
            g.record_stream(compute)   # zero_grad may release it while the side stream still reads it
            rc = L.halo_adamw_bf16_step_single(
                _lib.ptr(p), _lib.ptr(g), _lib.ptr(m_dev), _lib.ptr(v_dev), _lib.c_ll(n),
                ctypes.c_ulonglong(param_name_hash(name)), _lib.c_int(1 if gdtype == torch.float32 else 0),
                _lib.c_float(b1), _lib.c_float(b2), _lib.c_float(step_size), _lib.c_float(bc2_sqrt),
                _lib.c_float(eps), _lib.c_float(wd_factor), ctypes.c_ulonglong(self.key), ctypes.c_ulonglong(step),
                _lib.ptr(self._grad_scale), _lib.ptr(self._skip), ctypes.c_void_p(compute.cuda_stream),
            )
            _lib.check(rc, "halo_adamw_bf16_step_single")
            ev_done = torch.cuda.Event()
            ev_done.record(compute)
            self.ready_events[p] = ev_done
            d2h.wait_event(ev_done)
            with torch.cuda.stream(d2h):
                st["exp_avg"].copy_(m_dev, non_blocking=True)
                st["exp_avg_sq"].copy_(v_dev, non_blocking=True)
                self._slot_free[slot].record(d2h)
        if self._grad_scale is not None:
            self._grad_scale.record_stream(compute)

    # ---- update on the host CPU ------------------------------------------------------------------------
    def _host_compute_step(self, on_host, device, b1, b2, step_size, bc2_sqrt, eps, wd_factor, step):
        """Gradient to the host, AdamWBF16 there (all cores), new weight back; one background thread keeps the
        copy of tensor i + 1, the update of tensor i and the return of tensor i - 1 going at the same time. The
        caller returns at once; consumers of a parameter wait in :meth:`wait_ready`."""
        self.join_host_worker()
        if self._cpu_streams is not None:
            self._cpu_streams[1].synchronize()      # last step's return copies have left the host weights
        main = torch.cuda.current_stream(device)
        # the host needs the clip coefficient and the skip verdict: one read per step, after the norm is final
        scale = float(self._grad_scale.item()) if self._grad_scale is not None else None
        if self._skip is not None and int(self._skip.item()):
            return
        if self._cpu_streams is None:
            self._cpu_streams = (torch.cuda.Stream(device), torch.cuda.Stream(device))
            biggest = max(p.numel() for _, p, _ in on_host)
            self._g_host = [_pinned_zeros(biggest, torch.bfloat16) for _ in range(2)]
        d2h, h2d = self._cpu_streams
        d2h.wait_stream(main)
        work = []
        for name, p, st in on_host:
            if "master" not in st:
                st["master"] = _pinned_zeros(p.numel(), torch.bfloat16)
                st["master"].copy_(p.detach().reshape(-1))            # once: the host keeps the weights it updates
            g = p.grad.contiguous()
            g.record_stream(d2h)
            flag = threading.Event()
            self._cpu_flags[p] = flag
            work.append((name, p, st, g, flag))
        hyper = (b1, b2, step_size, bc2_sqrt, eps, wd_factor, step, scale)
        self._worker = threading.Thread(target=self._host_worker, args=(work, hyper, device), daemon=True)
        self._worker.start()

    def _host_worker(self, work, hyper, device):
        b1, b2, step_size, bc2_sqrt, eps, wd_factor, step, scale = hyper
        torch.cuda.set_device(device)
        L = _lib.host_lib()
        d2h, h2d = self._cpu_streams
        out_events = [None, None]

        def fetch(i):
            _, p, _, g, _ = work[i]
            with torch.cuda.stream(d2h):
                self._g_host[i % 2][:p.numel()].copy_(g.reshape(-1), non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(d2h)
            return ev

        pending = fetch(0)
        for i, (name, p, st, g, flag) in enumerate(work):
            nxt = fetch(i + 1) if i + 1 < len(work) else None          # its slot was released by update i - 1
            pending.synchronize()
            n = p.numel()
            ptr = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
            L.halo_host_adamw_bf16(
                ptr(st["master"]), ptr(self._g_host[i % 2]), ptr(st["exp_avg"]), ptr(st["exp_avg_sq"]), ctypes.c_longlong(n),
                ctypes.c_ulonglong(param_name_hash(name)), ctypes.c_ulonglong(self.key), ctypes.c_ulonglong(step),
                ctypes.c_float(b1), ctypes.c_float(b2), ctypes.c_float(step_size), ctypes.c_float(bc2_sqrt), ctypes.c_float(eps),
                ctypes.c_float(wd_factor), ctypes.c_float(scale if scale is not None else 1.0),
                ctypes.c_int(0 if scale is None else 1), ctypes.c_int(0))
            with torch.cuda.stream(h2d):
                p.data.copy_(st["master"].view(p.shape), non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(h2d)
            self.ready_events[p] = ev
            flag.set()
            work[i] = (name, p, st, None, flag)                        # the gradient may be freed now
            pending = nxt

    def join_host_worker(self) -> None:
        if self._worker is not None:
            self._worker.join()
            self._worker = None

    def wait_ready(self, params, stream=None) -> None:
        """Make ``stream`` (default: the current one) wait for the streamed updates of ``params``."""
        if not self.ready_events and not self._cpu_flags:
            return
        stream = stream or torch.cuda.current_stream()
        for p in params:
            flag = self._cpu_flags.pop(p, None)
            if flag is not None:
                flag.wait()                       # the host thread has issued this parameter's return copy
            ev = self.ready_events.pop(p, None)
            if ev is not None:
                stream.wait_event(ev)

    def wait_all_ready(self) -> None:
        self.wait_ready(list(dict.fromkeys(list(self._cpu_flags) + list(self.ready_events))))

    def synchronize_state(self) -> None:
        """Wait until every moment written by the last step has landed in host memory (call before
        reading the state, e.g. to save a checkpoint)."""
        self.join_host_worker()
        if self._cpu_streams is not None:
            for s in self._cpu_streams:
                s.synchronize()
        if self._streams is not None:
            self._opt_stream.synchronize()
            for s in self._streams:
                s.synchronize()

    def state_bytes_on_host(self) -> int:
        total = 0
        for st in self.state.values():
            if st.get("host_state"):
                total += 2 * st["exp_avg"].numel() * 2
        return total

    @staticmethod
    def expected_step_seconds(host_bytes: int, pcie_gbs: float = 50.0) -> float:
        """Lower bound of the streamed part of a step: every moment crosses PCIe once each way,
        both directions concurrently."""
        return host_bytes / (pcie_gbs * 1e9) if host_bytes else 0.0


