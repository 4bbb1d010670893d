"""External reward sources behind one contract: an LLM judge, a reward-model endpoint and the White Circle policy check.

A scorer grades samples for ONE reward term. ``score`` never raises for a sample - a request that failed comes back as a
``ScoreResult`` with ``score=None`` and the ``error`` - and ``verify`` makes one real request in the run's shape, so a bad
endpoint or key fails the launch instead of every episode. Requests are plain ``urllib`` calls run on worker threads
under a per-term concurrency bound; a timeout, a transport error, 408 / 429 and 5xx are retried with exponential
backoff or the server's ``Retry-After`` (capped), any other status fails at once.

A sample is a mapping with ``prompt`` and ``completion``, each either a string or a list of chat messages
(``{"role", "content", "tool_calls"?, "name"?, "tool_call_id"?}``).

(The roles of halo/rewards/scorers/{base,judge,reward_model,whitecircle}.py.)"""

from __future__ import annotations

import asyncio
import json
import os
import re
import time
import urllib.error
import urllib.request
import uuid
from dataclasses import dataclass, field

from .terms import JudgeTerm, PolicyCheckTerm, RewardModelTerm

TRANSIENT_STATUS = frozenset({408, 429})
MAX_RETRY_AFTER_S = 60.0
MAX_EVENTS_PER_REQUEST = 50            # the policy-check API's cap on the events of one request
POLICY_API_VERSION = "2026-06-01"
POLICY_API_KEY_VARIABLE = "WHITECIRCLE_API_KEY"
CHECKLIST_FLAG_CONFIDENCE = 0.5
_PROBE = {"prompt": [{"role": "user", "content": "Reply with the single word: ready"}],
          "completion": [{"role": "assistant", "content": "ready"}]}


@dataclass(frozen=True)
class ScoreResult:
    score: float | None                 # in [0, 1]; None with ``error`` when no verdict was reached
    metrics: dict = field(default_factory=dict)
    error: str | None = None
    detail: str | None = None
    veto: bool = False                  # a judge's fired veto check: the episode loses its other credits too


class HttpError(RuntimeError):
    def __init__(self, status: int, body: str):
        super().__init__(f"status {status}: {body[:200]}")
        self.status = status


def post_json(url: str, body: dict, headers: dict | None = None, timeout: float = 30.0, max_retries: int = 4,
              retry_wait: float = 1.0, sleep=time.sleep) -> dict:
    """POST ``body`` as JSON and return the decoded reply, retrying what is worth retrying."""
    data = json.dumps(body).encode()
    for attempt in range(max_retries + 1):
        wait = retry_wait * 2 ** attempt
        req = urllib.request.Request(url, data=data, method="POST",
                                     headers={"Content-Type": "application/json", **(headers or {})})
        try:
            with urllib.request.urlopen(req, timeout=timeout) as resp:
                return json.loads(resp.read().decode() or "{}")
        except urllib.error.HTTPError as e:
            text = e.read().decode(errors="replace")
            if not (e.code in TRANSIENT_STATUS or e.code >= 500) or attempt == max_retries:
                raise HttpError(e.code, text) from None
            try:
                wait = min(max(float(e.headers.get("Retry-After")), 0.0), MAX_RETRY_AFTER_S)
            except (TypeError, ValueError):
                pass
        except (urllib.error.URLError, TimeoutError, ConnectionError):
            if attempt == max_retries:
                raise
        sleep(wait)
    raise RuntimeError("retries exhausted")      # not reached: the last attempt returns or raises


def as_messages(part, role: str) -> list[dict]:
    if isinstance(part, str):
        return [{"role": role, "content": part}]
    return [dict(m) for m in (part or [])]


def content_text(content) -> str:
    """A message's text: the string itself, or the text parts of a list-of-parts content."""
    if content is None:
        return ""
    if isinstance(content, str):
        return content
    return "".join(p.get("text", "") for p in content if isinstance(p, dict) and p.get("type", "text") == "text")


class Scorer:
    """Base: bounded concurrency, per-sample isolation of failures, the launch probe."""

    def __init__(self, term):
        self.term = term
        self._sem = None
        self._sem_loop = None

    def score_one_sync(self, sample) -> ScoreResult:      # pragma: no cover - the subclasses' job
        raise NotImplementedError

    async def score_one(self, sample) -> ScoreResult:
        try:
            return await asyncio.to_thread(self.score_one_sync, sample)
        except Exception as e:  # noqa: BLE001 - a failed request is a result, never an exception of the round
            return ScoreResult(None, error=f"{type(self).__name__} failed: {type(e).__name__}: {e}")

    async def _bounded(self, sample) -> ScoreResult:
        loop = asyncio.get_running_loop()
        if self._sem is None or self._sem_loop is not loop:      # a semaphore belongs to the loop that first used it
            self._sem, self._sem_loop = asyncio.Semaphore(max(1, getattr(self.term, "max_concurrency", 8))), loop
        async with self._sem:
            return await self.score_one(sample)

    async def score(self, samples) -> list[ScoreResult]:
        return list(await asyncio.gather(*(self._bounded(s) for s in samples)))

    async def verify(self) -> None:
        result = await self.score_one(_PROBE)
        if result.score is None:
            raise RuntimeError(f"reward term {self.term.name!r}: launch probe failed: {result.error}")

    async def __call__(self, term, episode) -> float:
        """The callable form the composer takes: a failed request raises here and is counted there."""
        result = await self._bounded(episode)
        if result.score is None:
            raise RuntimeError(result.error)
        return result.score


_JSON_OBJECT = re.compile(r"\{.*\}", re.S)


class JudgeScorer(Scorer):
    """An OpenAI-compatible chat endpoint grades the completion against the term's rubric and answers with a JSON object
    ``{"score": 0..1, "veto": bool?, "reason": str?}`` (text around the object is tolerated)."""

    def __init__(self, term: JudgeTerm, base_url: str, api_key: str | None = None, **http):
        super().__init__(term)
        self.url = base_url.rstrip("/") + "/v1/chat/completions"
        self.headers = {"Authorization": f"Bearer {api_key}"} if api_key else {}
        self.http = http

    def request_body(self, sample) -> dict:
        convo = as_messages(sample.get("prompt"), "user") + as_messages(sample.get("completion"), "assistant")
        shown = "\n".join(f"[{m['role']}] {content_text(m.get('content'))}" for m in convo)
        ask = (f"Rubric:\n{self.term.rubric}\n\nConversation:\n{shown}\n\nGrade the LAST assistant turn against the rubric. "
               'Answer with one JSON object: {"score": <number from 0 to 1>, "veto": <true|false>, "reason": "<short>"}')
        return {"model": self.term.model, "temperature": 0.0, "messages": [{"role": "user", "content": ask}]}

    def score_one_sync(self, sample) -> ScoreResult:
        reply = post_json(self.url, self.request_body(sample), self.headers, **self.http)
        text = content_text(reply["choices"][0]["message"].get("content"))
        found = _JSON_OBJECT.search(text)
        if not found:
            raise ValueError(f"the grading model's reply holds no JSON object: {text[:120]!r}")
        verdict = json.loads(found.group(0))
        score = float(verdict["score"])
        if not 0.0 <= score <= 1.0:
            raise ValueError(f"the grading model's score {score} is outside [0, 1]")
        return ScoreResult(score, {f"{self.term.name}/score": score}, detail=verdict.get("reason"), veto=bool(verdict.get("veto", False)))


class RewardModelScorer(Scorer):
    """A reward-model service: POST ``{"messages": [...]}`` to the term's endpoint, read ``{"score": x}`` (or the first of
    ``{"scores": [...]}``). ``logistic=True`` maps an unbounded logit into (0, 1)."""

    def __init__(self, term: RewardModelTerm, logistic: bool = False, **http):
        super().__init__(term)
        self.logistic = logistic
        self.http = http

    def score_one_sync(self, sample) -> ScoreResult:
        messages = as_messages(sample.get("prompt"), "user") + as_messages(sample.get("completion"), "assistant")
        reply = post_json(self.term.endpoint, {"messages": messages}, **self.http)
        raw = float(reply["score"] if "score" in reply else reply["scores"][0])
        if self.logistic:
            import math

            raw = 1.0 / (1.0 + math.exp(-raw))
        if not 0.0 <= raw <= 1.0:
            raise ValueError(f"reward-model score {raw} is outside [0, 1] (pass logistic=True for a logit)")
        return ScoreResult(raw, {f"{self.term.name}/score": raw})


def conversation_events(sample, final_only: bool = False) -> tuple[list[dict], list[str]]:
    """The conversation as the policy-check API's events, in order, each with an ``event_id``; and the ids of the
    policy's own events (its text and its tool calls' arguments): the verdict reads those, every earlier event is
    their context. ``final_only`` reads the last assistant message alone."""
    prompt = as_messages(sample.get("prompt"), "user")
    completion = as_messages(sample.get("completion"), "assistant")
    events, own = [], []
    last_assistant = max((i for i, m in enumerate(completion) if m.get("role") == "assistant"), default=-1)
    for index, m in enumerate(prompt + completion):
        role, text = m.get("role"), content_text(m.get("content"))
        if role == "tool":
            items = [{"type": "tool", "name": m.get("name"), "call_id": m.get("tool_call_id"), "output": text}]
        else:
            items = [{"type": "message", "role": role, "content": text}] if text else []
        for call in m.get("tool_calls") or []:
            fn = call.get("function", call)
            args = fn.get("arguments")
            if isinstance(args, str):
                try:
                    args = json.loads(args)
                except ValueError:
                    args = {"raw": args}
            items.append({"type": "tool", "name": fn.get("name"), "call_id": call.get("id"), "arguments": args or {}})
        mine = role == "assistant" and index >= len(prompt) and (not final_only or index - len(prompt) == last_assistant)
        for item in items:
            item["event_id"] = f"e{len(events)}"
            events.append(item)
            if mine:
                own.append(item["event_id"])
    return events, own


class PolicyCheckScorer(Scorer):
    """The White Circle API as a scorer: the completion, in its conversation, checked against the policies of the term's
    environment over ``POST /api/events``. One request per sample (no completion is checked in another's conversation);
    a conversation of more than 50 events goes in consecutive requests under one session id. The key is read from
    ``WHITECIRCLE_API_KEY`` when the scorer is built and lives only in its headers."""

    def __init__(self, term: PolicyCheckTerm, base_url: str | None = None, **http):
        super().__init__(term)
        key = os.environ.get(POLICY_API_KEY_VARIABLE, "").strip()
        if not key:
            raise RuntimeError(f"reward term {term.name!r}: no API key - set {POLICY_API_KEY_VARIABLE}")
        self.url = (base_url or f"https://{term.region}.whitecircle.com").rstrip("/") + "/api/events"
        self.headers = {"Authorization": f"Bearer {key}", "whitecircle-version": POLICY_API_VERSION}
        self.http = {"timeout": term.request_timeout, "max_retries": term.max_retries, "retry_wait": term.retry_wait, **http}

    def score_one_sync(self, sample) -> ScoreResult:
        events, own = conversation_events(sample, final_only=self.term.view == "final")
        flagged_key = f"{self.term.name}/flagged"
        if not own:
            # no text and no call violates nothing, and full credit for it would teach the policy to say nothing
            return ScoreResult(0.0, {flagged_key: 0.0}, detail="empty completion")
        session, results = uuid.uuid4().hex, {}
        for start in range(0, len(events), MAX_EVENTS_PER_REQUEST):
            body = {"environment_id": self.term.environment_id, "external_session_id": session,
                    "events": events[start:start + MAX_EVENTS_PER_REQUEST]}
            reply = post_json(self.url, body, self.headers, **self.http)
            for kind in reply.values():
                if isinstance(kind, list):
                    results.update({r["event_id"]: r for r in kind if isinstance(r, dict) and "event_id" in r})
        return self.verdict([results.get(e) for e in own])

    def verdict(self, results) -> ScoreResult:
        """Raises when an event of the completion has no verdict, when no policy was checked on any of them, or when a
        listed policy was checked on none of them (a silent pass would be full credit for nothing)."""
        term = self.term
        for r in results:
            if r is None:
                raise ValueError("the reply carries no result for an event of the completion")
            if r.get("status") != "completed" or r.get("flagged") is None:
                raise ValueError(f"no verdict (status {r.get('status')!r}): {r.get('note')}")
        violated, names = {}, {}
        for r in results:
            for policy, outcome in (r.get("policies") or {}).items():
                violated[policy] = violated.get(policy, False) or bool(outcome.get("flagged"))
                names[policy] = outcome.get("name", policy)
        if not violated:
            raise ValueError(f"no policy was checked on the completion: {results[0].get('note')}")
        listed = term.checklist or term.policies
        if listed:
            unchecked = [p for p in listed if p not in violated]
            if unchecked:
                raise ValueError(f"policies {unchecked} were not checked on the completion: no condition selected them")
            read = {p: violated[p] for p in listed}       # a listed term reads its own policies only
            score = 1.0 - sum(read.values()) / len(read)
        else:
            read = violated
            score = 0.0 if any(r["flagged"] for r in results) else 1.0
        broken = [names[p] for p, hit in read.items() if hit]
        flagged_key = f"{term.name}/flagged"
        if term.checklist:
            confidence = 1.0 - score
            return ScoreResult(score, {flagged_key: float(confidence >= CHECKLIST_FLAG_CONFIDENCE), f"{term.name}/confidence": confidence},
                               detail=f"confidence {confidence:.2f}: {', '.join(broken)}" if broken else None)
        metrics = {flagged_key: float(score < 1.0)}
        if term.policies:
            metrics.update({f"{term.name}/{p}": float(hit) for p, hit in read.items()})
        return ScoreResult(score, metrics, detail=f"flagged: {', '.join(broken)}" if broken else None)


def route_by_term(scorers: dict):
    """One composer callable over several scorers of a kind: ``scorers`` maps term names to their scorer."""
    async def call(term, episode) -> float:
        return await scorers[term.name](term, episode)
    return call


async def verify_all(scorers) -> None:
    """The launch probe of every external scorer, together; the first failure names its term."""
    await asyncio.gather(*(s.verify() for s in scorers))
