"""On-policy self-distillation beside GRPO (SDPG): ``L = L_GRPO + beta(k) * L_OPD``.

The teacher is the policy itself, without gradient, reading the same completion after a prompt that also reveals the
gold answer (a "hint"); the on-policy distillation term pulls the student's next-token distribution at every completion
token toward that privileged teacher's (reverse KL by default), only on rollouts whose advantage is strictly positive
(a tied or unscorable group expressed no preference to pull toward). ``beta(k)`` ramps up over the first steps and decays
to zero over the last.

On packed rows: a round's micro-batch is one packed stream of ``[prompt, completion]`` rows; the teacher's rows
``[prompt, hint, completion]`` form a second packed stream of the same micro-batch, and two index vectors pair each
scored completion position of the student stream with the position of the teacher stream that predicts the same token.
Both streams run through the model once; the vocabulary-sized distributions are formed chunk by chunk from the gathered
hidden states, so no ``[tokens, vocab]`` tensor outlives a chunk. The student's hidden states feed the GRPO surrogate and
the distillation term from one forward and one backward.

The term's denominator is the round's gated token count summed over micro-batches and data-parallel ranks, like the
surrogate's, so its scale depends neither on the token budget nor on the data-parallel width.

Counterpart of halo/trainers/distillation/sdpg.py:1-250 and halo/trainers/distillation/opd_term.py.
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from halo_b200.data.packing import pack_documents
from halo_b200.trainers.distillation import chunked_kd_sum
from halo_b200.trainers.grpo.trainer import GRPOBatch, GRPOTrainer, Rollout, counted_completion_tokens

HINT_TEMPLATE = "\n(The reference answer is: {answer})\n"


def render_hint(template: str, answer) -> str | None:
    """The hint text, or None when the row has no answer (the teacher then reads the plain prompt)."""
    if answer is None or (isinstance(answer, str) and not answer.strip()):
        return None
    import string

    fields = {f for _, f, _, _ in string.Formatter().parse(template) if f}
    if fields - {"answer"}:
        raise ValueError(f"the hint template may only name {{answer}}, not {sorted(fields - {'answer'})}")
    return template.format(answer=answer)


def beta_schedule(step: int, total_steps: int, base: float, warmup_steps: int = 0, decay_steps: int = 0) -> float:
    """``base`` with a linear ramp from 0 over the first ``warmup_steps`` and a linear decay to 0 over the last
    ``decay_steps`` of ``total_steps``."""
    beta = base
    if warmup_steps > 0 and step < warmup_steps:
        beta = base * (step + 1) / warmup_steps
    if decay_steps > 0 and total_steps > 0 and step >= total_steps - decay_steps:
        beta = min(beta, base * max(total_steps - step - 1, 0) / decay_steps)
    return float(beta)


@dataclass
class OPDPlan:
    """The teacher stream of one micro-batch and the pairing of positions."""
    input_ids: torch.Tensor          # [Tt]
    position_ids: torch.Tensor       # [Tt]
    cu_seqlens: np.ndarray
    student_idx: torch.Tensor        # [N] positions of the student stream whose next token is a policy-produced completion token
    teacher_idx: torch.Tensor        # [N] the teacher stream's position predicting the same token
    gate: torch.Tensor               # [N] 1.0 where the row's advantage allows the term
    denominator: float = 0.0

    def to(self, device):
        mv = lambda t: t.to(device, non_blocking=True)  # noqa: E731
        return OPDPlan(mv(self.input_ids), mv(self.position_ids), self.cu_seqlens, mv(self.student_idx), mv(self.teacher_idx),
                       mv(self.gate), self.denominator)


def build_opd_plan(rollouts: list[Rollout], student_cu, adv: torch.Tensor, positive_only: bool) -> OPDPlan:
    docs = []
    s_idx, t_idx, gate = [], [], []
    t_start = 0
    for i, r in enumerate(rollouts):
        tp = np.asarray(r.teacher_prompt_ids if r.teacher_prompt_ids is not None else r.prompt_ids)
        docs.append(np.concatenate([tp, r.completion_ids]))
        p, q, n = len(r.prompt_ids), len(tp), len(r.completion_ids)
        own = np.ones(n, bool) if r.completion_mask is None else np.asarray(r.completion_mask, bool)
        s0 = int(student_cu[i])
        js = np.nonzero(own)[0]
        s_idx.append(s0 + p - 1 + js)            # the position that predicts completion token j
        t_idx.append(t_start + q - 1 + js)
        allowed = (float(adv[i]) > 0) if positive_only else True
        gate.append(np.full(len(js), 1.0 if allowed else 0.0, np.float32))
        t_start += q + n
    packed = pack_documents(docs)
    cat = lambda parts, dt: torch.from_numpy(np.concatenate(parts).astype(dt)) if parts else torch.zeros(0, dtype=torch.int64)  # noqa: E731
    return OPDPlan(packed.input_ids, packed.position_ids, packed.cu_seqlens, cat(s_idx, np.int64), cat(t_idx, np.int64),
                   cat(gate, np.float32))


class SDPGTrainer(GRPOTrainer):
    """``GRPOTrainer`` with the on-policy distillation term. Rollouts carry ``teacher_prompt_ids`` (see
    :func:`attach_teacher_prompts`); a rollout without them distils from the teacher on the plain prompt."""

    def __init__(self, *args, sdpg_beta_base: float = 1.0, sdpg_beta_warmup_steps: int = 0, sdpg_beta_decay_steps: int = 0,
                 sdpg_loss: str = "reverse_kl", sdpg_temperature: float = 1.0, opd_positive_advantage_only: bool = True, **kw):
        if sdpg_loss not in ("reverse_kl", "forward_kl", "jsd"):
            raise ValueError(f"sdpg_loss must be reverse_kl, forward_kl or jsd, got {sdpg_loss!r}")
        if not (sdpg_temperature > 0 and np.isfinite(sdpg_temperature)):
            raise ValueError("sdpg_temperature must be finite and positive")
        if not (sdpg_beta_base >= 0 and np.isfinite(sdpg_beta_base)):
            raise ValueError("sdpg_beta_base must be finite and non-negative")
        self.sdpg = dict(base=sdpg_beta_base, warmup=sdpg_beta_warmup_steps, decay=sdpg_beta_decay_steps, loss=sdpg_loss,
                         temperature=sdpg_temperature, positive_only=opd_positive_advantage_only)
        self.last_opd = float("nan")
        self.last_beta = float("nan")
        super().__init__(*args, **kw)
        if getattr(self.grpo, "tree_packing", False) and sdpg_beta_base:
            raise ValueError("the distillation term pairs every completion with its own teacher row; tree packing stores "
                             "prompts once per group and is not combined with it (set sdpg_beta_base: 0 or tree_packing: false)")

    def plan_round(self, rollouts):
        batches = super().plan_round(rollouts)
        if not self.sdpg["base"]:
            return batches
        # the same advantages the parent used (recomputed: cheap and keeps the parent's interface unchanged)
        from halo_b200.trainers.grpo import advantages as adv_mod

        rewards = torch.tensor([r.reward for r in rollouts], dtype=torch.float32)
        adv, _ = adv_mod.group_advantages(rewards, self.grpo.num_generations, self.grpo.scale_rewards, self.grpo.std_floor)
        by_id = {id(r): i for i, r in enumerate(rollouts)}
        gated = 0.0
        for b in batches:
            rows = b.rollouts
            if any(id(r) not in by_id for r in rows):
                # a filler micro-batch: it still runs the teacher pass (every rank must enter the same collectives) and
                # pairs no position
                b.opd = build_opd_plan(rows, b.cu_seqlens, torch.zeros(len(rows)), True)
                continue
            idx = [by_id[id(r)] for r in rows]
            b.opd = build_opd_plan(rows, b.cu_seqlens, adv[idx], self.sdpg["positive_only"])
            gated += float(b.opd.gate.sum())
        denominator = max(self._world_sum(gated), 1.0)
        for b in batches:
            b.opd.denominator = denominator
        return batches

    def beta(self) -> float:
        total = int(getattr(self.args, "max_steps", 0) or 0)
        return beta_schedule(self.global_step, total, self.sdpg["base"], self.sdpg["warmup"], self.sdpg["decay"])

    def compute_loss(self, model, batch: GRPOBatch, normalizer):
        plan = getattr(batch, "opd", None)
        beta = self.beta() if self.sdpg["base"] else 0.0
        self.last_beta = beta
        if plan is None or beta == 0.0:
            return super().compute_loss(model, batch, normalizer)
        if model.cfg.final_logit_softcapping:
            raise NotImplementedError("the distillation term on soft-capped output logits is not built")
        dev = batch.input_ids.device
        plan = plan.to(dev)
        # one student forward: its hidden states feed the surrogate (through the parent) and the distillation term
        captured = {}
        inner_hidden = model.hidden_states

        def capturing(*a, **kw):
            h = inner_hidden(*a, **kw)
            captured["h"] = h
            return h

        model.hidden_states = capturing
        try:
            loss = super().compute_loss(model, batch, normalizer)
        finally:
            del model.hidden_states                   # the instance attribute shadows the method only for this call
        hs = captured["h"].reshape(-1, captured["h"].shape[-1])[plan.student_idx]
        was_training = model.training
        with torch.no_grad():
            ht_all = model.hidden_states(plan.input_ids, plan.position_ids, plan.cu_seqlens)
        model.train(was_training)
        ht = ht_all.reshape(-1, ht_all.shape[-1])[plan.teacher_idx]
        w = model.head_weight()
        opd_sum = chunked_kd_sum(hs, w, ht, w.detach(), plan.gate, self.sdpg["loss"], self.sdpg["temperature"])
        opd = opd_sum / plan.denominator
        self.last_opd = float(opd.detach())
        return loss + beta * opd

    def extra_logs(self) -> dict:
        logs = dict(super().extra_logs())
        logs.update({"sdpg/beta": self.last_beta, "sdpg/opd": self.last_opd})
        return logs


def attach_teacher_prompts(rollouts: list[Rollout], answers: list, tokenizer, template: str = HINT_TEMPLATE) -> int:
    """Give every rollout its privileged prompt: the prompt followed by the tokenised hint. ``answers`` align with
    ``rollouts`` (already repeated per generation). Returns how many rows had no answer."""
    if len(answers) != len(rollouts):
        raise RuntimeError(f"{len(answers)} answers for {len(rollouts)} rollouts: a teacher prompt would carry another row's answer")
    missing = 0
    for r, a in zip(rollouts, answers):
        hint = render_hint(template, a)
        if hint is None:
            missing += 1
            r.teacher_prompt_ids = None
            continue
        ids = tokenizer(hint, add_special_tokens=False)["input_ids"] if callable(tokenizer) else tokenizer.encode(hint)
        r.teacher_prompt_ids = np.concatenate([np.asarray(r.prompt_ids), np.asarray(ids, dtype=np.int64)])
    return missing


class HintedSource:
    """Wrap a rollout source whose prompts are task rows: after every round each rollout gets its privileged prompt from
    the task's ``answer_field``. Rows without an answer are counted (and logged once): their teacher reads the plain prompt,
    so the term degenerates to self-distillation there."""

    def __init__(self, source, tokenizer, answer_field: str = "answer", template: str = HINT_TEMPLATE):
        render_hint(template, "probe")               # a bad template fails at construction, on every rank alike
        self.source, self.tokenizer, self.answer_field, self.template = source, tokenizer, answer_field, template
        self.rows_without_answer = 0
        self._warned = False

    def __getattr__(self, name):
        return getattr(self.source, name)

    def __call__(self, round_index: int):
        rollouts = self.source(round_index)
        if rollouts is None:
            return None
        tasks = getattr(self.source, "last_tasks", None)
        if tasks is None or len(tasks) != len(rollouts):
            raise RuntimeError("the rollout source does not report the task row of every rollout (last_tasks): the hint "
                               "needs each row's gold answer")
        answers = [(t or {}).get(self.answer_field) for t in tasks]
        missing = attach_teacher_prompts(rollouts, answers, self.tokenizer, self.template)
        self.rows_without_answer += missing
        if missing and not self._warned:
            import logging

            self._warned = True
            logging.getLogger(__name__).warning("%d rollout rows carry no %r value: their teacher runs on the plain prompt",
                                                missing, self.answer_field)
        return rollouts


__all__ = ["SDPGTrainer", "HintedSource", "OPDPlan", "build_opd_plan", "beta_schedule", "render_hint", "attach_teacher_prompts",
           "counted_completion_tokens"]
