"""Programming-task pool preparation (rating bounds, exclusions, unsound suites, constant-proof suites, per-band
hold-out) and offline re-grading of recorded episodes against a repaired suite."""

import json

import pytest

from halo_b200.entrypoints import code_tasks as C

_ADD = "a, b = map(int, input().split())\nprint(a + b)\n"


def _problem(pid, rating=1000, tests=None, **kw):
    tests = tests or [{"input": "1 2\n", "output": "3\n"}, {"input": "5 7\n", "output": "12\n"}]
    return {"id": pid, "statement": "add two numbers", "public_tests": tests[:1], "hidden_tests": tests, "rating": rating,
            "reference_solution": _ADD, **kw}


def test_prepare_drops_with_reasons_and_carves_a_holdout(tmp_path):
    rows = [_problem(f"p{i}", rating=800 + 100 * (i % 8)) for i in range(16)]
    rows.append(_problem("too_easy", rating=300))
    rows.append(_problem("unrated", rating=None))
    rows.append({k: v for k, v in _problem("no_rating_key").items() if k != "rating"})           # nothing to bound: kept
    rows.append(_problem("old_1"))
    rows.append(_problem("dup"))
    rows.append(_problem("dup"))
    rows.append(_problem("always_yes", tests=[{"input": "1\n", "output": "YES\n"}, {"input": "2\n", "output": "YES\n"}],
                         reference_solution="print('YES')\n"))
    rows.append(_problem("bad_suite", tests=[{"input": "1 2\n", "output": "3\n"}, {"input": "5 7\n", "output": "13\n"}]))
    excl = tmp_path / "exclude.txt"
    excl.write_text("# known leaks\nold_*\n\n")
    train, test, drops = C.prepare(rows, min_rating=500, max_rating=2000, exclusions=C.load_exclusions(str(excl)),
                                   per_band=1, width=400, first=800, seed=3)
    assert drops == {"rating outside the bounds (or unrated)": 2, "excluded by the list": 1, "no id or duplicate id": 1,
                     "a constant answer passes every hidden test": 1, "the reference solution fails its own tests": 1}
    ids = {r["id"] for r in train} | {r["id"] for r in test}
    assert ids == {f"p{i}" for i in range(16)} | {"no_rating_key", "dup"} and not {r["id"] for r in train} & {r["id"] for r in test}
    # bands of 400 from 800: [800, 1200) holds ratings 800..1100, [1200, 1600) holds 1200..1500; one row from each; the
    # two rows without a usable rating form a band of their own
    assert sorted(C.band_of(r["rating"], 400, 800) for r in test if "rating" in r) == [0, 1]
    assert all("reference_solution" not in r for r in train + test)
    again = C.prepare(rows, 500, 2000, C.load_exclusions(str(excl)), 1, 400, 800, seed=3)
    assert [r["id"] for r in again[1]] == [r["id"] for r in test]                                  # a seeded draw
    assert C.rating_in_bounds({"rating": None}, None, None) and not C.rating_in_bounds({"rating": None}, 0, None)
    assert C.suite_accepts_a_constant(_problem("x")) is None
    # the command line writes both splits
    src = tmp_path / "problems.jsonl"
    src.write_text("".join(json.dumps(r) + "\n" for r in rows))
    assert C.main(["prepare", str(src), "--out-dir", str(tmp_path / "pool"), "--min-rating", "500", "--exclude", str(excl),
                   "--holdout-per-band", "1"]) == 0
    assert len(C.read_jsonl(str(tmp_path / "pool" / "test.jsonl"))) >= 2


def test_regrade_against_a_repaired_suite(tmp_path):
    tasks = [C.to_task_row(_problem("a")), C.to_task_row(_problem("b"))]
    wrong = "a, b = map(int, input().split())\nprint(a * b)\n"
    episodes = [
        {"task": 0, "sample": 0, "score": 1.0, "task_id": "a", "turns": [{"role": "assistant", "content": f"```python\n{wrong}```"},
                                                                           {"role": "assistant", "content": f"fixed:\n```python\n{_ADD}```"}]},
        {"task": 0, "sample": 1, "score": 1.0, "task_id": "a", "turns": [{"role": "assistant", "content": f"```python\n{wrong}```"}]},
        {"task": 1, "sample": 0, "score": 0.0, "task_id": "b", "completion": f"```python\n{_ADD}```"},        # the older record form
        {"task": 1, "sample": 1, "score": 0.5, "task_id": "b", "turns": [{"role": "assistant", "content": "I give up"}]},
    ]
    report, rows = C.regrade({"env": "code", "options": {}}, episodes, tasks)
    assert [r["score"] for r in rows] == [1.0, 0.0, 1.0, 0.0] and [r["sent_a_program"] for r in rows] == [True, True, True, False]
    assert report["mean_score"] == 0.5 and report["recorded_mean_score"] == 0.625 and report["changed"] == 3
    assert report["pass@1"] == 0.5 and report["pass@2"] == 1.0
    assert rows[1]["hidden_passed"] == 0                      # 1 * 2 is not 3 and 5 * 7 is not 12
    partial = C.regrade({"env": "code", "options": {"all_or_nothing": "true"}}, episodes[:1], tasks)[1][0]
    assert partial["score"] == 1.0
    with pytest.raises(ValueError, match="lines up with"):
        C.regrade({}, [dict(episodes[0], task=1)], tasks)
    with pytest.raises(IndexError):
        C.regrade({}, [dict(episodes[0], task=5)], tasks)
    with pytest.raises(ValueError, match="only 'code' episodes"):
        C.regrade({"env": "qa"}, episodes, tasks)
    # through the files, with the meta line first
    ep_path, task_path = tmp_path / "episodes.jsonl", tmp_path / "tasks.jsonl"
    ep_path.write_text(json.dumps({"meta": {"env": "code", "options": {}}}) + "\n" + "".join(json.dumps(e) + "\n" for e in episodes))
    task_path.write_text("".join(json.dumps(t) + "\n" for t in tasks))
    assert C.main(["regrade", str(ep_path), "--tasks", str(task_path), "--out", str(tmp_path / "regraded.jsonl")]) == 0
    assert len(C.read_jsonl(str(tmp_path / "regraded.jsonl"))) == 4
