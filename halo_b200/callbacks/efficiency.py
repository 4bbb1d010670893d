"""Throughput and model-FLOPs utilisation from CUDA-event step boundaries
(halo/callbacks/efficiency.py:203-563, halo/callbacks/model_flops.py).

FLOPs per token = 6 * N_active (matrix parameters touched per token, forward + backward) plus the
attention-score term 12 * head_dim * n_heads * (mean attended keys per query) per layer; with full
recomputation the hardware does 8/6 of that, which is reported separately as HFU."""

from __future__ import annotations

import numpy as np
import torch

from halo_b200 import hardware
from halo_b200.trainers.base import Callback


def attended_keys(cu_seqlens) -> float:
    """Sum over documents of n(n+1)/2: causal (query, key) pairs in a packed row."""
    n = np.diff(np.asarray(cu_seqlens, dtype=np.float64))
    return float((n * (n + 1) / 2).sum())


def model_flops_per_step(cfg, cu_seqlens, n_tokens: int) -> float:
    counts = cfg.param_counts()
    dense = 6.0 * (counts["active"] - 0) * n_tokens
    from halo_b200.models.attention_cost import attention_flops

    return dense + attention_flops(cfg, cu_seqlens)        # per layer: windowed layers visit fewer keys


class EfficiencyCallback(Callback):
    def __init__(self, cfg, world_size: int = 1, peak_flops: float | None = None):
        self.cfg, self.world = cfg, world_size
        self.peak = peak_flops or hardware.peak_flops("bf16") or hardware.GPU_PEAK_FLOPS["B200"]["bf16"]
        self.measured = hardware.measured_peaks()
        self._last = None
        self._tokens = 0
        self._flops = 0.0
        self.history: list[dict] = []

    def on_train_begin(self, trainer):
        self._mark()

    def _mark(self):
        if torch.cuda.is_available():
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self._last = ev
        else:
            import time

            self._last = time.perf_counter()

    def on_batch(self, trainer, batch):
        # the ranks of a tensor-parallel group work on ONE row together: each accounts for its share of the tokens and
        # of the model FLOPs, so the per-GPU figures stay per GPU
        tp = getattr(getattr(trainer, "model", None), "tensor_parallel", None)
        # likewise the stages of a pipeline: a micro-batch passes through all of them
        stage = getattr(getattr(trainer, "engine", None), "stage", None)
        ways = max(1, int(getattr(tp, "size", 1) or 1)) * max(1, int(getattr(stage, "n_stages", 1) or 1))
        self.note_batch(batch, share=1.0 / ways)

    def note_batch(self, batch, share: float = 1.0):
        self._tokens += batch.n_tokens * share
        self._flops += model_flops_per_step(self.cfg, batch.cu_seqlens, batch.n_tokens) * share

    def on_log(self, trainer, logs):
        if self._last is None or "step_seconds" not in logs:
            return
        prev = self._last
        self._mark()
        if torch.cuda.is_available():
            torch.cuda.synchronize()
            seconds = prev.elapsed_time(self._last) / 1e3
        else:
            seconds = self._last - prev
        if seconds <= 0:
            return
        rec = {"tokens_per_s_per_gpu": self._tokens / seconds, "step": logs.get("step")}
        if self._flops:
            rec["mfu"] = self._flops / seconds / self.peak
            rec["mfu_of_measured"] = self._flops / seconds / (self.measured.bf16_tflops_sustained * 1e12)
        if torch.cuda.is_available():
            rec["peak_gib"] = torch.cuda.max_memory_allocated() / 2**30
        logs.update(rec)
        self.history.append(rec)
        self._tokens, self._flops = 0, 0.0
