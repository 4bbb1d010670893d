"""Checks of an external generation server before the first GRPO round. A server that is misconfigured for training
does not fail: it produces rollouts that train the wrong thing (truncated rows, log-probabilities of a different
distribution than the one sampled, re-tokenised text instead of the sampled tokens). Each check here turns one such
silent failure into a refusal (a list of reasons, raised together) or a logged warning, on the one rank that holds the
weight-sync client.

Checks:

* the server answers, and serves a model with the trainer's vocabulary size;
* its context window holds one rollout (``max_prompt_length + max_completion_length``);
* a sampled completion comes back with token ids and one log-probability per token (re-tokenised text is refused);
* with a temperature other than 1 the reported log-probabilities are those of the distribution actually sampled
  (temperature applied), measured on a greedy probe whose top-1 log-probability must change with the temperature;
* one idle sequence decodes fast enough that a full-length completion fits the request timeout;
* flags that change the served distribution relative to the trainer (quantised weights, speculative decoding)
  are reported, and quantised weights are refused unless allowed;
* the first weight push is accepted (the group forms and one small tensor round-trips a session).

Counterpart of halo/trainers/grpo/rollout/engine_preflight.py:83-815.
"""

from __future__ import annotations

import logging
import math
import time
from dataclasses import dataclass, field

log = logging.getLogger(__name__)

PROBE_PROMPT = [1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12]
RATE_PROBE_TOKENS = 64
DEADLINE_WARN_SHARE = 0.5
DEADLINE_REFUSE_MULTIPLE = 1.0


@dataclass
class PreflightReport:
    refusals: list[str] = field(default_factory=list)
    warnings: list[str] = field(default_factory=list)
    facts: dict = field(default_factory=dict)

    def raise_if_refused(self) -> None:
        for w in self.warnings:
            log.warning("rollout server preflight: %s", w)
        if self.refusals:
            raise ValueError("the rollout server cannot be used for training:\n  - " + "\n  - ".join(self.refusals))


def _complete(client, **payload) -> dict:
    body = {"model": client.model_id or (client.info.model_id if client.info else ""), **payload}
    return client.request("POST", "/v1/completions", json=body, timeout=120.0, retry=False).json()


def check_context_window(report: PreflightReport, info, max_prompt_length: int, max_completion_length: int) -> None:
    need = max_prompt_length + max_completion_length
    report.facts["max_model_len"] = info.max_model_len
    if info.max_model_len and need > info.max_model_len:
        report.refusals.append(
            f"its context window ({info.max_model_len}) is smaller than one rollout ({need} = max_prompt_length + "
            "max_completion_length): lower max_completion_length or serve a longer context")


def check_sampled_token_ids(report: PreflightReport, client) -> None:
    raw = _complete(client, prompt=PROBE_PROMPT, max_tokens=4, temperature=1.0, logprobs=0, return_tokens_as_token_ids=True)
    lp = raw["choices"][0].get("logprobs") or {}
    tokens, lps = lp.get("tokens") or [], lp.get("token_logprobs") or []
    if not tokens or not all(str(t).startswith("token_id:") for t in tokens):
        report.refusals.append("it does not return the sampled token ids with a completion (tokens come back as text); "
                               "re-tokenised text is not the sampled sequence, so importance ratios would be wrong")
    elif len(lps) != len(tokens) or any(x is None for x in lps):
        report.refusals.append("it does not return one log-probability per sampled token")


def check_temperature_semantics(report: PreflightReport, client, temperature: float) -> None:
    """The trainer divides its logits by ``temperature`` before comparing with the sampler's log-probabilities, so the
    server must report log-probabilities of the tempered distribution. Greedy probes at two temperatures: the top-1
    log-probability of the same first token must differ (it rises as the temperature falls)."""
    if temperature == 1.0:
        return
    tops = []
    for t in (1.0, temperature):
        raw = _complete(client, prompt=PROBE_PROMPT, max_tokens=1, temperature=t, top_k=1, logprobs=0, seed=0)
        lps = (raw["choices"][0].get("logprobs") or {}).get("token_logprobs") or [None]
        tops.append(lps[0])
    report.facts["top1_logprob_at_1_and_T"] = tops
    if tops[0] is None or tops[1] is None:
        report.warnings.append("could not read a top-1 log-probability to check how the temperature enters the reported values")
    elif abs(tops[0] - tops[1]) < 1e-6 and abs(tops[0]) > 1e-6:
        report.refusals.append(
            f"it reports log-probabilities of the untempered distribution while sampling at temperature {temperature}: "
            "the importance ratio would compare two different distributions (enable processed log-probabilities on the server)")


def probe_generation_rate(client) -> float | None:
    """Tokens per second of one idle sequence: the better of two timed completions (the first may warm a kernel)."""
    rates = []
    for _ in range(2):
        start = time.perf_counter()
        raw = _complete(client, prompt=PROBE_PROMPT, max_tokens=RATE_PROBE_TOKENS, temperature=0.0, ignore_eos=True)
        elapsed = time.perf_counter() - start
        n = (raw.get("usage") or {}).get("completion_tokens", 0)
        if n >= RATE_PROBE_TOKENS // 2 and elapsed > 0:
            rates.append(n / elapsed)
    return max(rates, default=None)


def check_turn_deadline(report: PreflightReport, client, max_completion_length: int, request_timeout_s: float) -> None:
    rate = probe_generation_rate(client)
    if rate is None:
        return
    needed = max_completion_length / rate
    report.facts["idle_tokens_per_s"] = rate
    advice = (f"a completion that runs to max_completion_length={max_completion_length} needs about {needed:.0f} s at the "
              f"{rate:.0f} tokens/s one idle sequence decodes, against a request timeout of {request_timeout_s:g} s (and a "
              f"sequence in a busy round decodes slower): raise the timeout to at least {math.ceil(2 * needed)} s or lower "
              "max_completion_length")
    if needed > DEADLINE_REFUSE_MULTIPLE * request_timeout_s:
        report.refusals.append("even idle it cannot finish a full completion inside the request timeout: " + advice)
    elif needed > DEADLINE_WARN_SHARE * request_timeout_s:
        report.warnings.append(advice)


def check_served_distribution(report: PreflightReport, info, allow_quantized: bool = False) -> None:
    flags = {str(k).lower(): v for k, v in (info.flags or {}).items()}
    quant = next((v for k, v in flags.items() if "quantization" in k and v not in (None, "", "None", "none")), None)
    if quant and not allow_quantized:
        report.refusals.append(f"it serves quantised weights ({quant}): pushed bf16 weights would be re-quantised and the sampler "
                               "would differ from the policy by more than the importance correction assumes")
    spec = next((v for k, v in flags.items() if "speculative" in k and v not in (None, "", "None", "none", False)), None)
    if spec:
        report.warnings.append(f"speculative decoding is on ({spec}): sampled tokens follow the target distribution only if "
                               "the server's acceptance rule is exact")


def check_vocabulary(report: PreflightReport, client, vocab_size: int) -> None:
    """Ask for the top log-probabilities at one position with an id beyond the trainer's vocabulary as prompt: a server with
    a smaller vocabulary refuses the request."""
    try:
        _complete(client, prompt=[max(vocab_size - 1, 0)], max_tokens=1, temperature=0.0)
    except Exception as exc:  # noqa: BLE001
        report.refusals.append(f"it rejects token id {vocab_size - 1}, the last id of the trainer's vocabulary ({exc}): "
                               "the served model has a different tokenizer")


def check_first_push(report: PreflightReport, client, device=None) -> None:
    """The transfer group forms and an empty update session opens and closes (no tensor is changed)."""
    try:
        client.begin_update(device)
        client.end_update()
        client.pushes = 0
    except Exception as exc:  # noqa: BLE001
        report.refusals.append(f"a weight update could not be opened: {exc}")


def run_preflight(client, model_cfg, grpo_args, request_timeout_s: float = 1800.0, device=None, push_probe: bool = True,
                  connection_timeout_s: float = 300.0) -> PreflightReport:
    client.check_server(total_timeout=connection_timeout_s)
    info = client.read_server_info()
    report = PreflightReport(facts={"version": info.version, "model_id": info.model_id, "world_size": info.world_size})
    check_context_window(report, info, grpo_args.max_prompt_length, grpo_args.max_completion_length)
    check_served_distribution(report, info)
    check_vocabulary(report, client, model_cfg.vocab_size)
    check_sampled_token_ids(report, client)
    check_temperature_semantics(report, client, grpo_args.temperature)
    check_turn_deadline(report, client, grpo_args.max_completion_length, request_timeout_s)
    if push_probe and not report.refusals:
        check_first_push(report, client, device)
    log.info("rollout server preflight: %s", report.facts)
    report.raise_if_refused()
    return report
