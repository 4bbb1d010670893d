"""External reward scorers against a local HTTP server that plays a judge model, a reward model and the policy-check API:
verdict arithmetic, retries on 429 / 5xx with Retry-After, per-sample failure isolation, the launch probe, chunking of
long conversations, and the composer wiring."""

import asyncio
import json
import threading
from http.server import BaseHTTPRequestHandler, HTTPServer

import pytest

from halo_b200.rewards import scorers as S
from halo_b200.rewards.terms import JudgeTerm, PolicyCheckTerm, RewardComposer, RewardModelTerm, parse_terms


class _Server:
    def __init__(self):
        outer = self
        self.requests, self.fail_next = [], []       # fail_next: list of (status, headers) served before real answers

        class H(BaseHTTPRequestHandler):
            def log_message(self, *a):
                pass

            def do_POST(self):
                body = json.loads(self.rfile.read(int(self.headers["Content-Length"])))
                outer.requests.append((self.path, {k.lower(): v for k, v in self.headers.items()}, body))
                if outer.fail_next:
                    status, headers = outer.fail_next.pop(0)
                    self.send_response(status)
                    for k, v in headers.items():
                        self.send_header(k, v)
                    self.end_headers()
                    self.wfile.write(b"busy")
                    return
                out = outer.answer(self.path, body)
                data = json.dumps(out).encode()
                self.send_response(200)
                self.send_header("Content-Length", str(len(data)))
                self.end_headers()
                self.wfile.write(data)

        self.httpd = HTTPServer(("127.0.0.1", 0), H)
        self.url = f"http://127.0.0.1:{self.httpd.server_address[1]}"
        threading.Thread(target=self.httpd.serve_forever, daemon=True).start()

    def answer(self, path, body):
        if path == "/v1/chat/completions":
            text = body["messages"][0]["content"]
            score = 0.25 if "wrong" in text else 1.0
            return {"choices": [{"message": {"content": f'Verdict: {{"score": {score}, "veto": {str("rude" in text).lower()}, "reason": "r"}} done'}}]}
        if path == "/rm":
            return {"score": 0.75 if "good" in body["messages"][-1]["content"] else 0.1}
        if path == "/api/events":
            results = []
            for e in body["events"]:
                text = json.dumps(e)
                pol = {"p_spam": {"flagged": "buy now" in text, "name": "No spam"}, "p_pii": {"flagged": "ssn" in text, "name": "No PII"}}
                results.append({"event_id": e["event_id"], "status": "completed", "flagged": any(p["flagged"] for p in pol.values()),
                                "policies": pol})
            return {"messages": [r for r, e in zip(results, body["events"]) if e["type"] == "message"],
                    "tools": [r for r, e in zip(results, body["events"]) if e["type"] == "tool"]}
        return {}

    def close(self):
        self.httpd.shutdown()


@pytest.fixture()
def server():
    s = _Server()
    yield s
    s.close()


def test_judge_and_reward_model(server):
    judge = S.JudgeScorer(JudgeTerm("helpful", rubric="be right", model="judge-1"), server.url, api_key="k", retry_wait=0.01)
    good, bad, rude = asyncio.run(judge.score([{"prompt": "2+2?", "completion": "4"}, {"prompt": "2+2?", "completion": "wrong 5"},
                                               {"prompt": "hi", "completion": "rude reply"}]))
    assert good.score == 1.0 and bad.score == 0.25 and rude.veto and not good.veto
    path, headers, body = server.requests[0]
    assert path == "/v1/chat/completions" and headers["authorization"] == "Bearer k" and body["model"] == "judge-1"
    assert "be right" in body["messages"][0]["content"] and "[assistant] 4" in body["messages"][0]["content"]
    rm = S.RewardModelScorer(RewardModelTerm("rm", endpoint=server.url + "/rm"), retry_wait=0.01)
    assert [r.score for r in asyncio.run(rm.score([{"prompt": "q", "completion": "good"}, {"prompt": "q", "completion": "meh"}]))] == [0.75, 0.1]
    asyncio.run(S.verify_all([judge, rm]))
    # a dead endpoint: the sample gets an error, not an exception; the launch probe raises by name
    dead = S.RewardModelScorer(RewardModelTerm("rm2", endpoint="http://127.0.0.1:9/rm"), max_retries=0, timeout=0.5)
    res = asyncio.run(dead.score([{"prompt": "q", "completion": "a"}]))[0]
    assert res.score is None and "RewardModelScorer failed" in res.error
    with pytest.raises(RuntimeError, match="'rm2': launch probe failed"):
        asyncio.run(dead.verify())


def test_retries_follow_retry_after_and_stop_on_client_errors(server):
    waits = []
    server.fail_next = [(429, {"Retry-After": "7"}), (503, {}), (500, {"Retry-After": "900"})]
    out = S.post_json(server.url + "/rm", {"messages": [{"role": "assistant", "content": "good"}]}, retry_wait=0.5, sleep=waits.append)
    assert out == {"score": 0.75} and waits == [7.0, 1.0, 60.0]                  # the server's wait, the backoff, the cap
    server.fail_next = [(404, {})]
    with pytest.raises(S.HttpError, match="status 404"):
        S.post_json(server.url + "/rm", {}, sleep=waits.append)
    assert len(waits) == 3                                                        # a 404 is not retried
    server.fail_next = [(500, {})] * 3
    with pytest.raises(S.HttpError, match="status 500"):
        S.post_json(server.url + "/rm", {}, max_retries=2, retry_wait=0.0, sleep=waits.append)


def test_policy_check(server, monkeypatch):
    monkeypatch.delenv(S.POLICY_API_KEY_VARIABLE, raising=False)
    with pytest.raises(RuntimeError, match="no API key"):
        S.PolicyCheckScorer(PolicyCheckTerm("wc", environment_id="env"))
    monkeypatch.setenv(S.POLICY_API_KEY_VARIABLE, "secret")
    convo = {"prompt": [{"role": "system", "content": "be nice"}, {"role": "user", "content": "sell me something"}],
             "completion": [{"role": "assistant", "content": "", "tool_calls": [{"id": "c1", "function": {"name": "lookup", "arguments": '{"q": "ssn 123"}'}}]},
                            {"role": "tool", "name": "lookup", "tool_call_id": "c1", "content": "buy now"},      # the tool's text is context, not the policy's
                            {"role": "assistant", "content": "here is a fair offer"}]}
    events, own = S.conversation_events(convo)
    assert [e["type"] for e in events] == ["message", "message", "tool", "tool", "message"] and own == ["e2", "e4"]
    assert events[2]["arguments"] == {"q": "ssn 123"} and S.conversation_events(convo, final_only=True)[1] == ["e4"]
    plain = S.PolicyCheckScorer(PolicyCheckTerm("wc", environment_id="env", retry_wait=0.01), base_url=server.url)
    r = asyncio.run(plain.score([convo]))[0]
    assert r.score == 0.0 and r.metrics == {"wc/flagged": 1.0} and r.detail == "flagged: No PII"
    _, headers, body = server.requests[-1]
    assert headers["authorization"] == "Bearer secret" and headers["whitecircle-version"] == S.POLICY_API_VERSION
    assert body["environment_id"] == "env" and len(body["external_session_id"]) == 32
    final = S.PolicyCheckScorer(PolicyCheckTerm("wc", environment_id="env", view="final"), base_url=server.url)
    assert asyncio.run(final.score([convo]))[0].score == 1.0                       # the last turn alone is clean
    listed = S.PolicyCheckScorer(PolicyCheckTerm("wc", environment_id="env", policies=["p_spam", "p_pii"]), base_url=server.url)
    r = asyncio.run(listed.score([convo]))[0]
    assert r.score == 0.5 and r.metrics == {"wc/flagged": 1.0, "wc/p_spam": 0.0, "wc/p_pii": 1.0}
    check = S.PolicyCheckScorer(PolicyCheckTerm("wc", environment_id="env", checklist=["p_spam", "p_pii"]), base_url=server.url)
    r = asyncio.run(check.score([convo]))[0]
    assert r.score == 0.5 and r.metrics == {"wc/flagged": 1.0, "wc/confidence": 0.5}
    unknown = S.PolicyCheckScorer(PolicyCheckTerm("wc", environment_id="env", policies=["p_other"]), base_url=server.url)
    assert "were not checked" in asyncio.run(unknown.score([convo]))[0].error
    silent = asyncio.run(plain.score([{"prompt": "hi", "completion": [{"role": "assistant", "content": ""}]}]))[0]
    assert silent.score == 0.0 and silent.detail == "empty completion"
    # a conversation of 120 events goes in three requests under one session id
    long = {"prompt": [{"role": "user", "content": f"turn {i}"} for i in range(119)], "completion": "fine"}
    n0 = len(server.requests)
    assert asyncio.run(plain.score([long]))[0].score == 1.0
    sent = server.requests[n0:]
    assert [len(b["events"]) for _, _, b in sent] == [50, 50, 20] and len({b["external_session_id"] for _, _, b in sent}) == 1
    with pytest.raises(ValueError, match="not both"):
        PolicyCheckTerm("wc", environment_id="env", policies=["a"], checklist=["b"])
    with pytest.raises(ValueError, match="environment_id"):
        parse_terms([{"type": "whitecircle"}])


def test_composer_settles_every_external_term(server, monkeypatch):
    monkeypatch.setenv(S.POLICY_API_KEY_VARIABLE, "secret")
    terms = parse_terms([{"type": "grader", "grader": "exact_match", "name": "right", "weight": 1.0},
                         {"type": "judge", "name": "helpful", "rubric": "r", "model": "m", "weight": 0.5},
                         {"type": "reward_model", "name": "rm", "endpoint": server.url + "/rm", "weight": 2.0},
                         {"type": "whitecircle", "name": "safe", "environment_id": "env", "weight": 1.0}])
    composer = RewardComposer(terms,
                              judge=S.route_by_term({"helpful": S.JudgeScorer(terms[1], server.url)}),
                              reward_model=S.route_by_term({"rm": S.RewardModelScorer(terms[2])}),
                              policy_check=S.route_by_term({"safe": S.PolicyCheckScorer(terms[3], base_url=server.url)}))
    total, parts = composer.score({"prompt": "q", "completion": "good", "target": "good"})
    assert parts == {"right": 1.0, "helpful": 1.0, "rm": 0.75, "safe": 1.0} and total == pytest.approx(1.0 + 0.5 + 1.5 + 1.0)
    assert composer.failures == 0
