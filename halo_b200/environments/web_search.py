"""A web-search tool for tool-using environments: one function tool (``web_search(query, max_results)``) over a
search API, with a per-episode call budget, a result cache (the same query inside a round is answered once), bounded
request time and results rendered as a short numbered list the policy can cite.

Providers: ``brave`` (``GET https://api.search.brave.com/res/v1/web/search``, key in ``BRAVE_API_KEY``), ``tavily``
(``POST https://api.tavily.com/search``, key in ``TAVILY_API_KEY``), or ``custom`` (any endpoint that answers
``{"results": [{"title", "url", "snippet"}]}`` to ``GET ?q=...&n=...``). There is no network on the build machines: the
tests run the tool against a local endpoint of the ``custom`` shape.

Counterpart of halo/environments/tools/web_search.py:1-242 and the budgeting of halo/environments/tools/accounting.py.
"""

from __future__ import annotations

import json
import os
import threading
import urllib.parse
import urllib.request

from .protocols import ToolRegistry

REQUEST_TIMEOUT_S = 20.0
MAX_SNIPPET_CHARS = 300


class SearchBudgetExceeded(RuntimeError):
    pass


class WebSearch:
    def __init__(self, provider: str = "brave", endpoint: str = "", api_key: str = "", max_calls: int = 8, max_results: int = 5,
                 timeout_s: float = REQUEST_TIMEOUT_S, opener=None):
        if provider not in ("brave", "tavily", "custom"):
            raise ValueError(f"unknown search provider {provider!r}; choose brave, tavily or custom")
        self.provider, self.endpoint = provider, endpoint
        self.api_key = api_key or os.environ.get({"brave": "BRAVE_API_KEY", "tavily": "TAVILY_API_KEY"}.get(provider, ""), "")
        if provider != "custom" and not self.api_key:
            raise PermissionError(f"the {provider} search provider needs its API key in the environment")
        if provider == "custom" and not endpoint:
            raise ValueError("the custom search provider needs an endpoint")
        self.max_calls, self.max_results, self.timeout_s = max_calls, max_results, timeout_s
        self._open = opener or urllib.request.urlopen
        self._cache: dict = {}
        self._lock = threading.Lock()
        self.calls = 0

    def reset_budget(self) -> None:
        self.calls = 0

    # ---- providers -------------------------------------------------------------------------------------
    def _request(self, query: str, n: int) -> list[dict]:
        if self.provider == "brave":
            url = "https://api.search.brave.com/res/v1/web/search?" + urllib.parse.urlencode({"q": query, "count": n})
            req = urllib.request.Request(url, headers={"X-Subscription-Token": self.api_key, "Accept": "application/json"})
            raw = json.load(self._open(req, timeout=self.timeout_s))
            return [{"title": r.get("title", ""), "url": r.get("url", ""), "snippet": r.get("description", "")}
                    for r in (raw.get("web") or {}).get("results", [])]
        if self.provider == "tavily":
            body = json.dumps({"api_key": self.api_key, "query": query, "max_results": n}).encode()
            req = urllib.request.Request("https://api.tavily.com/search", data=body, headers={"Content-Type": "application/json"})
            raw = json.load(self._open(req, timeout=self.timeout_s))
            return [{"title": r.get("title", ""), "url": r.get("url", ""), "snippet": r.get("content", "")} for r in raw.get("results", [])]
        url = self.endpoint + ("&" if "?" in self.endpoint else "?") + urllib.parse.urlencode({"q": query, "n": n})
        raw = json.load(self._open(urllib.request.Request(url), timeout=self.timeout_s))
        return list(raw.get("results", []))

    # ---- the tool --------------------------------------------------------------------------------------
    def search(self, query: str, max_results: int = 0) -> str:
        query = " ".join(str(query).split())
        if not query:
            return "error: empty query"
        n = min(max_results or self.max_results, self.max_results)
        with self._lock:
            if self.calls >= self.max_calls:
                raise SearchBudgetExceeded(f"the search budget of {self.max_calls} calls per episode is used up")
            self.calls += 1
            cached = self._cache.get((query, n))
        if cached is None:
            try:
                cached = self._request(query, n)[:n]
            except Exception as exc:  # noqa: BLE001 - a failed search is an observation
                return f"error: the search failed ({type(exc).__name__}: {exc})"
            with self._lock:
                self._cache[(query, n)] = cached
        if not cached:
            return f"no results for {query!r}"
        lines = []
        for i, r in enumerate(cached, 1):
            snippet = " ".join(str(r.get("snippet", "")).split())[:MAX_SNIPPET_CHARS]
            lines.append(f"[{i}] {r.get('title', '').strip()} - {r.get('url', '')}\n    {snippet}")
        return "\n".join(lines)

    def register(self, registry: ToolRegistry, name: str = "web_search") -> None:
        registry.register(name, "Search the web; returns a numbered list of titles, URLs and snippets.",
                          {"query": {"type": "string", "description": "what to search for"},
                           "max_results": {"type": "integer", "description": f"at most {self.max_results}", "optional": True}},
                          self.search)
