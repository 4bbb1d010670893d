"""Pipeline parallelism: contiguous decoder-layer ranges on consecutive stage ranks, micro-batches run on a
1F1B (or GPipe) schedule, activations and their gradients travel between neighbours as point-to-point
messages of the process group (NCCL send/recv on GPUs, gloo on CPU).

The reference builds this on ``torch.distributed.pipelining`` (halo/distributed/pipeline_parallel/runner.py:26,
183-191; stage.py:342-410; partition.py:83-137; stage_losses.py:44-61). Here the schedule is a short explicit
loop, because a stage of this framework is just a ``Qwen3Model`` built with a layer range: the first stage owns
the embedding, the last one the final norm, the head and the fused loss. Packed rows have a fixed length, so
every message has the same shape ``[row_len, hidden]`` and needs no shape handshake.

Every rank of a pipeline replica reads the same micro-batches (token ids on the first stage, labels on the
last, positions and document boundaries everywhere).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist

from halo_b200.ops.cross_entropy import fused_linear_cross_entropy
from halo_b200.ops.norm import rms_norm


def partition_layers(n_layers: int, n_stages: int, head_weight: float = 1.0, embed_weight: float = 0.0,
                     split: list[int] | None = None) -> list[tuple[int, int]]:
    """Layer range of every stage. The last stage also runs the vocabulary head, which costs about
    ``head_weight`` decoder layers, the first the embedding (``embed_weight``); the split evens out
    layers + extras. ``split``: explicit first-layer index of stages 1.. (overrides the balance)."""
    if n_stages < 1 or n_layers < n_stages:
        raise ValueError(f"cannot cut {n_layers} layers into {n_stages} stages")
    if split:
        cuts = [0] + list(split) + [n_layers]
        if len(cuts) != n_stages + 1 or any(b <= a for a, b in zip(cuts, cuts[1:])):
            raise ValueError(f"pipeline_split {split} does not describe {n_stages} non-empty stages of {n_layers} layers")
        return list(zip(cuts[:-1], cuts[1:]))
    # stage s ends where the running cost (embedding + layers so far) reaches (s + 1) equal shares
    per = (n_layers + head_weight + embed_weight) / n_stages
    ranges, lo = [], 0
    for s in range(n_stages):
        if s == n_stages - 1:
            hi = n_layers
        else:
            hi = round((s + 1) * per - embed_weight)
            hi = max(hi, lo + 1)                              # never an empty stage
            hi = min(hi, n_layers - (n_stages - s - 1))       # leave a layer for every later stage
        ranges.append((lo, hi))
        lo = hi
    return ranges


@dataclass
class _InFlight:
    x_in: torch.Tensor | None
    out: torch.Tensor


class PipelineStage:
    """One stage's slice of the model plus its neighbours in the pipeline group."""

    def __init__(self, model, group, row_len: int, dtype=None, up_group=None):
        """``group`` carries the activations down the pipeline; ``up_group`` (same ranks, its own communicator) the
        gradients back up. On NCCL the point-to-point operations of one communicator run in the order they were
        issued, and a send only finishes once its receive has started: in the steady state of 1F1B stage s issues
        send(activation k+1), recv(gradient k) while stage s+1 issues send(gradient k), recv(activation k+1) - with one
        communicator each stage's send waits behind the other's, for ever. Two communicators let the two directions
        progress independently. ``up_group=None`` uses ``group`` for both (gloo, whose sends are buffered, and
        forward-only use)."""
        self.model, self.group = model, group
        self.up_group = up_group if up_group is not None else group
        self.n_stages = dist.get_world_size(group)
        self.stage = dist.get_rank(group)
        self.is_first, self.is_last = self.stage == 0, self.stage == self.n_stages - 1
        p = next(model.parameters())
        self.device, self.dtype = p.device, dtype or p.dtype
        self.shape = (row_len, model.cfg.hidden_size)
        self._pending: list = []
        self.prev = None if self.is_first else dist.get_global_rank(group, self.stage - 1) if group is not None else self.stage - 1
        self.next = None if self.is_last else dist.get_global_rank(group, self.stage + 1) if group is not None else self.stage + 1

    # ---- messages ------------------------------------------------------------------------------
    def _recv(self, src: int, up: bool = False) -> torch.Tensor:
        t = torch.empty(self.shape, dtype=self.dtype, device=self.device)
        dist.recv(t, src=src, group=self.up_group if up else self.group)
        return t

    def _send(self, t: torch.Tensor, dst: int, up: bool = False) -> None:
        # never a blocking send: in the steady state a stage sends an activation down while its neighbour sends
        # a gradient up, and two blocking sends facing each other would wait for ever
        t = t.contiguous()
        self._pending.append((dist.isend(t, dst=dst, group=self.up_group if up else self.group), t))

    def drain(self) -> None:
        for work, _ in self._pending:
            work.wait()
        self._pending.clear()

    # ---- one micro-batch ---------------------------------------------------------------------------
    def forward_micro(self, batch, normalizer) -> _InFlight:
        m = self.model
        ctx = m.make_context(batch.position_ids.reshape(-1), batch.cu_seqlens)
        if self.is_first:
            x_in = None
            x = m.embed(batch.input_ids)
        else:
            x_in = self._recv(self.prev).requires_grad_(True)
            x = x_in
        x = m.run_layers(x, ctx)
        if self.is_last:
            h = rms_norm(x, m.norm, m.cfg.rms_norm_eps)
            if m.cfg.final_logit_softcapping:
                out = m._capped_cross_entropy(h, batch.labels.reshape(-1), normalizer)
            else:
                out = fused_linear_cross_entropy(h, m.head_weight(), batch.labels.reshape(-1), normalizer)
        else:
            out = x
            self._send(out.detach(), self.next)
        return _InFlight(x_in, out)

    def backward_micro(self, fl: _InFlight) -> None:
        if self.is_last:
            fl.out.backward()
        else:
            g = self._recv(self.next, up=True)
            torch.autograd.backward(fl.out, g)
        if not self.is_first:
            self._send(fl.x_in.grad, self.prev, up=True)


def run_schedule(stage: PipelineStage, micro_batches: list, normalizer, schedule: str = "1f1b") -> torch.Tensor:
    """Forward + backward of every micro-batch; gradients accumulate in the stage's parameters. Returns the summed
    loss (a real value on the last stage, broadcast to the others afterwards by :func:`broadcast_loss`)."""
    M, S, s = len(micro_batches), stage.n_stages, stage.stage
    if schedule not in ("1f1b", "gpipe"):
        raise ValueError(f"unknown pipeline schedule {schedule!r}")
    warmup = M if schedule == "gpipe" else min(S - s - 1, M)
    inflight: list[_InFlight] = []
    losses = []
    f = b = 0

    def fwd():
        nonlocal f
        fl = stage.forward_micro(micro_batches[f], normalizer)
        if stage.is_last:
            losses.append(fl.out.detach())
        inflight.append(fl)
        f += 1

    def bwd():
        nonlocal b
        stage.backward_micro(inflight.pop(0))
        b += 1

    for _ in range(warmup):
        fwd()
    while f < M:                       # steady state: one forward, one backward
        fwd()
        bwd()
    while b < M:
        bwd()
    stage.drain()
    total = torch.stack(losses).sum() if losses else torch.zeros((), device=stage.device)
    return total.float()


@torch.no_grad()
def forward_only(stage: PipelineStage, batch, normalizer) -> torch.Tensor:
    """One micro-batch through the stages without a backward (evaluation): the last stage returns the loss, the others
    zero."""
    fl = stage.forward_micro(batch, normalizer)
    stage.drain()
    return fl.out.detach().float() if stage.is_last else torch.zeros((), device=stage.device)


def broadcast_loss(stage: PipelineStage, loss: torch.Tensor) -> torch.Tensor:
    """The last stage's loss, on every stage (for logging and the non-finite guard)."""
    t = loss.detach().clone().reshape(1).float()
    src = dist.get_global_rank(stage.group, stage.n_stages - 1) if stage.group is not None else stage.n_stages - 1
    dist.broadcast(t, src=src, group=stage.group)
    return t[0]


def stage_layer_range(cfg, stage: int, n_stages: int, split: list[int] | None = None) -> tuple[int, int]:
    """Decoder layers ``[lo, hi)`` of one stage. ``split``: explicit first-layer indices of stages 1.. or, as the
    configuration spells it, the layer COUNT of every stage."""
    if split and len(split) == n_stages:                  # per-stage layer counts -> first-layer indices of stages 1..
        starts, acc = [], 0
        for n in split[:-1]:
            acc += int(n)
            starts.append(acc)
        if acc + int(split[-1]) != cfg.num_hidden_layers:
            raise ValueError(f"pipeline_split {split} does not add up to {cfg.num_hidden_layers} layers")
        split = starts
    head_weight = (cfg.vocab_size * cfg.hidden_size) / max(1, cfg.param_counts()["active"] / cfg.num_hidden_layers) * 0.5
    return partition_layers(cfg.num_hidden_layers, n_stages, head_weight=min(head_weight, 4.0), split=split)[stage]


def build_stage_model(cfg, stage: int, n_stages: int, device, dtype=None, transport=None, seed: int = 0,
                      gradient_checkpointing: bool = True, split: list[int] | None = None):
    """The stage's model slice, initialised so that the union of all stages equals the unsplit model built with
    the same seed (initialisation is keyed by parameter name and global layer index)."""
    from halo_b200.models.qwen3 import build_model

    lo, hi = stage_layer_range(cfg, stage, n_stages, split)
    return build_model(cfg, device=device, dtype=dtype, transport=transport, seed=seed,
                       gradient_checkpointing=gradient_checkpointing, layer_range=(lo, hi), has_embed=stage == 0,
                       has_head=stage == n_stages - 1)
