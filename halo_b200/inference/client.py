"""Async OpenAI-compatible chat client and resumable parallel batch requests with a JSONL store
(halo/inference/*.py). Uses aiohttp directly; a request that fails is retried with backoff, a batch that is
interrupted resumes from the records already on disk."""

from __future__ import annotations

import asyncio
import json
import os
from dataclasses import asdict, dataclass, field


@dataclass
class ResponseRecord:
    request_id: str
    text: str = ""
    finish_reason: str = ""
    prompt_tokens: int = 0
    completion_tokens: int = 0
    error: str = ""
    raw: dict = field(default_factory=dict)


class ChatClient:
    def __init__(self, base_url: str, model: str, api_key: str = "", timeout_s: float = 600.0, max_retries: int = 4,
                 transport=None):
        self.base_url, self.model, self.api_key = base_url.rstrip("/"), model, api_key
        self.timeout_s, self.max_retries = timeout_s, max_retries
        self._transport = transport          # async callable(url, payload, headers) -> dict ; tests inject a fake

    async def _post(self, url: str, payload: dict, headers: dict) -> dict:
        if self._transport is not None:
            return await self._transport(url, payload, headers)
        import aiohttp

        async with aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=self.timeout_s)) as session:
            async with session.post(url, json=payload, headers=headers) as resp:
                resp.raise_for_status()
                return await resp.json()

    async def chat(self, request_id: str, messages: list[dict], **sampling) -> ResponseRecord:
        payload = {"model": self.model, "messages": messages, **sampling}
        headers = {"Authorization": f"Bearer {self.api_key}"} if self.api_key else {}
        delay = 0.5
        last = ""
        for attempt in range(self.max_retries + 1):
            try:
                raw = await self._post(f"{self.base_url}/chat/completions", payload, headers)
                choice = raw["choices"][0]
                usage = raw.get("usage", {})
                return ResponseRecord(request_id, choice["message"].get("content") or "", choice.get("finish_reason", ""),
                                      usage.get("prompt_tokens", 0), usage.get("completion_tokens", 0), raw=raw)
            except Exception as exc:  # noqa: BLE001 - any transport error is retried, then recorded
                last = f"{type(exc).__name__}: {exc}"
                if attempt < self.max_retries:
                    await asyncio.sleep(delay)
                    delay = min(delay * 2, 8.0)
        return ResponseRecord(request_id, error=last)


def load_done(store_path: str) -> dict[str, ResponseRecord]:
    done = {}
    if os.path.isfile(store_path):
        with open(store_path) as f:
            for line in f:
                try:
                    d = json.loads(line)
                except json.JSONDecodeError:
                    continue                     # a torn last line from an interrupted run
                if not d.get("error"):
                    done[d["request_id"]] = ResponseRecord(**d)
    return done


async def run_batch(client: ChatClient, requests: list[tuple[str, list[dict]]], store_path: str, concurrency: int = 32,
                    **sampling) -> dict[str, ResponseRecord]:
    """Every ``(request_id, messages)`` not already answered in ``store_path`` is sent; each answer is appended
    to the store as soon as it arrives, so an interrupted batch loses at most the requests in flight."""
    done = load_done(store_path)
    todo = [(rid, m) for rid, m in requests if rid not in done]
    sem = asyncio.Semaphore(concurrency)
    lock = asyncio.Lock()
    os.makedirs(os.path.dirname(store_path) or ".", exist_ok=True)

    async def one(rid, messages):
        async with sem:
            rec = await client.chat(rid, messages, **sampling)
        async with lock:
            with open(store_path, "a") as f:
                d = asdict(rec)
                d.pop("raw")
                f.write(json.dumps({**d, "raw": {}}) + "\n")
        if not rec.error:
            done[rid] = rec

    await asyncio.gather(*(one(rid, m) for rid, m in todo))
    return done
