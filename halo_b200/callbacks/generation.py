"""Callbacks that read the model through its own sampler or its multi-token-prediction head:

* :class:`GenerateExamplesCallback` - every ``every`` steps sample a few fixed prompts greedily and log the
  completions (decoded when a tokenizer is given), so a run's text can be eyeballed beside its loss
  (halo/callbacks/generate_examples.py). Skipped, with the reason logged once, where the model is sharded in a way
  the sampler does not serve.
* :class:`MtpAcceptanceGate` - the held-out gate of a head-only fit: draft acceptance on fixed held-out rows before
  the first step and at the end; a fit that did not gain ``min_gain`` fails the run, because loss and acceptance can
  fall together under an oversized learning rate (halo/callbacks/mtp.py:33-60).
* :class:`PhaseTimerCallback` - per-phase seconds from :class:`halo_b200.diagnostics.phase_timers.PhaseTimers` into
  the log records (halo/callbacks/phase_timer_callback.py).
"""

from __future__ import annotations

import logging

import numpy as np
import torch

from halo_b200.trainers.base import Callback

log = logging.getLogger(__name__)


class GenerateExamplesCallback(Callback):
    def __init__(self, prompts: list, every: int = 100, max_new_tokens: int = 64, tokenizer=None, eos_token_id=None):
        self.prompts = [np.asarray(p, dtype=np.int64) for p in prompts]
        self.every, self.max_new, self.tokenizer, self.eos = every, max_new_tokens, tokenizer, eos_token_id
        self.history: list[dict] = []
        self._skip_reason = None

    def _sample(self, trainer):
        from halo_b200.inference.generate import Generator, SamplingParams

        try:
            gen = Generator(trainer.model, eos_token_id=self.eos)
        except ValueError as exc:
            if self._skip_reason is None:
                self._skip_reason = str(exc)
                log.warning("example generations are skipped: %s", exc)
            return None
        was_training = trainer.model.training
        outs = gen.generate(self.prompts, SamplingParams(max_new_tokens=self.max_new, temperature=0.0))
        trainer.model.train(was_training)
        return outs

    def on_step_end(self, trainer, logs):
        if not self.every or trainer.global_step % self.every or not trainer.is_main:
            return
        outs = self._sample(trainer)
        if outs is None:
            return
        rows = []
        for o in outs:
            text = self.tokenizer.decode(o.token_ids.tolist(), skip_special_tokens=True) if self.tokenizer is not None else None
            rows.append({"prompt_ids": o.prompt_ids.tolist(), "completion_ids": o.token_ids.tolist(), "completion": text,
                         "finish_reason": o.finish_reason})
            log.info("step %d example: %s", trainer.global_step, text if text is not None else o.token_ids.tolist())
        self.history.append({"step": trainer.global_step, "examples": rows})


class MtpGateFailed(RuntimeError):
    pass


class MtpAcceptanceGate(Callback):
    def __init__(self, held_out_batches: list, min_gain: float = 0.0):
        self.batches, self.min_gain = held_out_batches, min_gain
        self.baseline = self.final = None

    @torch.no_grad()
    def acceptance(self, trainer) -> float:
        from halo_b200.models.mtp import draft_acceptance, shifted_targets

        model = trainer.model
        accepted = scored = 0
        for b in self.batches:
            b = b.to(trainer.device)
            ctx = model.make_context(b.position_ids.reshape(-1), b.cu_seqlens)
            states = model.mtp_states(model.trunk_states(b.input_ids, ctx), b.input_ids, ctx)
            a, s = draft_acceptance(states, model.head_weight(), shifted_targets(b.labels, b.cu_seqlens))
            accepted, scored = accepted + int(a), scored + int(s)
        return accepted / max(scored, 1)

    def on_train_begin(self, trainer):
        if trainer.model.mtp is None:
            raise ValueError("the acceptance gate needs a model with a multi-token-prediction head")
        self.baseline = self.acceptance(trainer)
        log.info("held-out draft acceptance before the fit: %.4f", self.baseline)

    def on_train_end(self, trainer):
        self.final = self.acceptance(trainer)
        log.info("held-out draft acceptance after the fit: %.4f (before: %.4f)", self.final, self.baseline)
        if self.final < self.baseline + self.min_gain:
            raise MtpGateFailed(f"held-out draft acceptance went from {self.baseline:.4f} to {self.final:.4f}, short of the "
                                f"required gain of {self.min_gain}: the fitted head is rejected (the last checkpoint holds it)")


class PhaseTimerCallback(Callback):
    """Adds ``phase/<name>`` seconds since the previous log to every log record."""

    def __init__(self, timers):
        self.timers = timers

    def on_log(self, trainer, logs):
        for name, seconds in self.timers.collect().items():
            logs[f"phase/{name}"] = seconds
