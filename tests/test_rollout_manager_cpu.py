"""The worker-pool rollout manager and the web-search tool (no network: local stand-ins)."""

import json
import os
import threading
from http.server import BaseHTTPRequestHandler, HTTPServer

import pytest


def scripted_policy(url, cfg):
    """A policy for the QA environment: answers with the task's question reversed, crashes its worker on request."""

    async def generate(messages, tools):
        from halo_b200.environments.base import Turn

        q = messages[-1]["content"]
        if "CRASH" in q and not os.path.exists(q.split("CRASH:")[1].strip()):
            open(q.split("CRASH:")[1].strip(), "w").write("x")        # die once: the retry finds the marker and answers
            os._exit(3)
        if "RAISE" in q:
            raise RuntimeError("server said no")
        return Turn("assistant", "\\boxed{4}" if "2+2" in q else f"{url}|{q[::-1]}")

    return generate


def test_manager_plays_rounds_in_order_and_survives_a_dying_worker(tmp_path):
    from halo_b200.environments.rollout_manager import RolloutConfig, RolloutManager

    cfg = RolloutConfig(env_type="qa", episode_timeout_s=60.0, max_retries=1)
    mgr = RolloutManager(cfg, ["http://a", "http://b"], n_workers=2, policy_factory=scripted_policy)
    try:
        marker = str(tmp_path / "crashed_once")
        tasks = [{"question": "what is 2+2", "answer": "4"}, {"question": f"CRASH:{marker}", "answer": "x"},
                 {"question": "RAISE", "answer": "y"}, {"question": "abc", "answer": "zzz"}]
        records = mgr.play(tasks)
        assert [r is not None for r in records] == [True] * 4
        assert records[0].score == 1.0
        assert os.path.exists(marker) and not records[1].done_reason.startswith("failed")     # retried on a fresh worker
        assert records[2].done_reason.startswith("failed: RuntimeError: server said no") and records[2].score == 0.0
        assert records[3].turns[0].content.endswith("|cba")
        # a second round works on the replaced pool, and both URLs were used
        again = mgr.play([{"question": f"q{i}", "answer": "?"} for i in range(6)])
        urls = {r.turns[0].content.split("|")[0] for r in again}
        assert urls == {"http://a", "http://b"}
    finally:
        mgr.close()


def test_engine_pauses_do_not_count_against_an_episode_deadline():
    import time

    from halo_b200.environments.rollout_manager import EnginePauseClock

    clock = EnginePauseClock()
    clock.begin()
    time.sleep(0.05)
    assert clock.paused_seconds() >= 0.05
    clock.end()
    total = clock.paused_seconds()
    time.sleep(0.02)
    assert clock.paused_seconds() == total


class _Search(BaseHTTPRequestHandler):
    hits = 0

    def log_message(self, *a):
        pass

    def do_GET(self):
        from urllib.parse import parse_qs, urlsplit

        type(self).hits += 1
        q = parse_qs(urlsplit(self.path).query)
        n = int(q["n"][0])
        results = [{"title": f"Result {i} for {q['q'][0]}", "url": f"http://x/{i}", "snippet": "word " * 200} for i in range(10)][:n]
        body = json.dumps({"results": results if "nothing" not in q["q"][0] else []}).encode()
        self.send_response(200)
        self.send_header("Content-Length", str(len(body)))
        self.end_headers()
        self.wfile.write(body)


def test_web_search_tool_budget_cache_and_rendering():
    from halo_b200.environments.protocols import ToolCall, ToolRegistry
    from halo_b200.environments.web_search import SearchBudgetExceeded, WebSearch

    server = HTTPServer(("127.0.0.1", 0), _Search)
    threading.Thread(target=server.serve_forever, daemon=True).start()
    try:
        ws = WebSearch("custom", endpoint=f"http://127.0.0.1:{server.server_address[1]}/search", max_calls=3, max_results=2)
        reg = ToolRegistry()
        ws.register(reg)
        out = reg.call(ToolCall("web_search", {"query": "  blackwell   tensor memory "}, "c1"))
        assert out.startswith("[1] Result 0 for blackwell tensor memory - http://x/0") and "[2]" in out and "[3]" not in out
        assert max(len(line) for line in out.splitlines()) <= 320
        assert reg.call(ToolCall("web_search", {"query": "blackwell tensor memory"}, "c2")) == out and _Search.hits == 1   # cached
        assert reg.call(ToolCall("web_search", {"query": "nothing here"}, "c3")).startswith("no results")
        assert "SearchBudgetExceeded" in reg.call(ToolCall("web_search", {"query": "one more"}, "c4"))
        ws.reset_budget()
        assert "error" not in reg.call(ToolCall("web_search", {"query": "one more"}, "c5"))
        with pytest.raises(SearchBudgetExceeded):
            ws.calls = 3
            ws.search("x")
    finally:
        server.shutdown()
    with pytest.raises(PermissionError):
        WebSearch("brave", api_key="")
