"""Host-side RL plumbing: graders, reward terms, environments, episode loop, endpoint client (CPU)."""

import asyncio
import json

import pytest

from halo_b200.environments import Turn, make_environment
from halo_b200.environments.episode_loop import play_episode
from halo_b200.environments.registry import environment_types
from halo_b200.environments.tasks import verdict
from halo_b200.inference.client import ChatClient, run_batch
from halo_b200.rewards import graders
from halo_b200.rewards.terms import RewardComposer, parse_terms


def test_graders():
    assert graders.last_boxed(r"so \boxed{\frac{1}{2}} and then \boxed{ 42 }") == " 42 "
    assert graders.boxed_accuracy(r"the answer is \boxed{1,000.0}", "1000") == 1.0
    assert graders.boxed_accuracy("1000", "1000", strict=True) == 0.0
    assert graders.boxed_accuracy("1000", "1000", strict=False) == 1.0
    assert graders.think_answer_format("<think>hm</think> 4") == 1.0 and graders.think_answer_format("4") == 0.0
    assert verdict("1 2\n3", "1  2 3\n") and not verdict("1 2", "1 2", "float") is False
    assert verdict("0.5", "0.50000001", "float") and not verdict("a", "b")


def test_terms_parse_and_compose():
    with pytest.raises(ValueError, match="unknown type"):
        parse_terms([{"type": "nope"}])
    with pytest.raises(ValueError, match="unknown grader"):
        parse_terms([{"type": "grader", "grader": "nope"}])
    terms = parse_terms([{"type": "grader", "grader": "boxed_accuracy", "weight": 1.0},
                         {"type": "format", "pattern": r".*\\boxed\{.*\}.*", "weight": 0.2},
                         {"type": "judge", "name": "style", "weight": 0.5, "exponent": 2.0}])

    async def judge(term, episode):
        return 0.5

    total, parts = RewardComposer(terms, judge=judge).score({"completion": r"\boxed{7}", "target": "7"})
    assert parts == {"grader_0": 1.0, "format_1": 1.0, "style": 0.5}
    assert abs(total - (1.0 + 0.2 + 0.5 * 0.25)) < 1e-9

    async def broken(term, episode):
        raise RuntimeError("judge down")

    comp = RewardComposer(terms, judge=broken)
    total, parts = comp.score({"completion": r"\boxed{7}", "target": "7"})
    assert parts["style"] == 0.0 and comp.failures == 1


def test_qa_and_code_episodes():
    assert {"qa", "code"} <= set(environment_types())

    async def answer(messages, tools):
        return Turn("assistant", r"It is \boxed{4}.")

    rec = asyncio.run(play_episode(make_environment("qa", {"question": "2+2?", "answer": "4"}), answer))
    assert rec.score == 1.0 and rec.done_reason == "answered"

    task = {"statement": "Print the sum of two integers.", "public_tests": [{"input": "1 2\n", "output": "3\n"}],
            "hidden_tests": [{"input": "5 7\n", "output": "12"}, {"input": "-1 1\n", "output": "0"}]}
    attempts = iter(["no code here", "```python\nprint(0)\n```", "```python\na,b=map(int,input().split())\nprint(a+b)\n```"])

    async def coder(messages, tools):
        return Turn("assistant", next(attempts))

    rec = asyncio.run(play_episode(make_environment("code", task, sandbox="subprocess"), coder))
    assert rec.score == 1.0 and rec.info["hidden_passed"] == 2 and len(rec.turns) == 3


def test_resumable_batch(tmp_path):
    calls = []

    async def fake(url, payload, headers):
        calls.append(payload["messages"][0]["content"])
        if payload["messages"][0]["content"] == "bad" and len([c for c in calls if c == "bad"]) < 2:
            raise ConnectionError("boom")
        return {"choices": [{"message": {"content": payload["messages"][0]["content"].upper()}, "finish_reason": "stop"}],
                "usage": {"prompt_tokens": 1, "completion_tokens": 1}}

    client = ChatClient("http://x/v1", "m", transport=fake, max_retries=2)
    store = str(tmp_path / "out.jsonl")
    reqs = [(f"r{i}", [{"role": "user", "content": c}]) for i, c in enumerate(["a", "bad", "c"])]
    done = asyncio.run(run_batch(client, reqs, store))
    assert {k: v.text for k, v in done.items()} == {"r0": "A", "r1": "BAD", "r2": "C"}
    n = len(calls)
    done = asyncio.run(run_batch(client, reqs, store))           # everything is on disk: nothing is sent again
    assert len(calls) == n and len(done) == 3
    assert all(json.loads(l)["request_id"] for l in open(store))


def test_offline_reward_scoring_resumes(tmp_path, capsys):
    import json

    from halo_b200.entrypoints import reward_scoring

    rows = tmp_path / "rows.jsonl"
    rows.write_text("\n".join(json.dumps({"completion": f"so \\boxed{{{i}}}", "target": str(i if i % 2 else -1)}) for i in range(6)))
    terms = tmp_path / "terms.yaml"
    terms.write_text("reward_terms:\n  - {type: grader, grader: boxed_accuracy, weight: 2.0}\n")
    out = tmp_path / "scored.jsonl"
    assert reward_scoring.main(["score", str(rows), "--terms", str(terms), "--out", str(out)]) == 0
    first = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert first["scored"] == 6 and first["mean_reward"] == 1.0            # three of six right, weight 2
    scored = [json.loads(l) for l in open(out)]
    assert [r["reward"] for r in scored] == [0.0, 2.0, 0.0, 2.0, 0.0, 2.0]
    out.write_text("\n".join(json.dumps(r) for r in scored[:4]) + "\n")     # an interrupted run left four rows
    assert reward_scoring.main(["score", str(rows), "--terms", str(terms), "--out", str(out)]) == 0
    again = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert again["scored"] == 2 and again["skipped"] == 4 and len(open(out).read().splitlines()) == 6
