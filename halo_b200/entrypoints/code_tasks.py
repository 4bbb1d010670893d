"""Offline work on programming tasks (the ``code`` environment): preparing a pool of problems, and re-grading recorded
episodes.

    python -m halo_b200.entrypoints.code_tasks prepare problems.jsonl --out-dir pool/ [--min-rating 800 --max-rating 2000]
                                               [--exclude ids.txt] [--holdout-per-band 20 --band-width 400] [--seed 0]
    python -m halo_b200.entrypoints.code_tasks regrade episodes.jsonl --tasks pool/test.jsonl [--out regraded.jsonl]

``prepare`` turns raw problem rows (``id``, ``statement``, ``public_tests``, ``hidden_tests``, optional ``rating``,
``reference_solution``, ``comparator``) into the rows the environment trains on, dropping - each with a counted reason -
rows outside the rating bounds (a row that has a ``rating`` key but no value is unrated and dropped; a row without the
key has nothing to bound), rows an exclusion list names (one id per line, a trailing ``*`` excludes the prefix), rows
whose reference solution does not pass their own tests (an unsound suite or checker), and rows whose hidden tests a
constant answer passes everywhere (a suite that accepts one expected output for every input teaches printing it). A
hold-out of ``--holdout-per-band`` problems is carved from every rating band (and from the rows below the first band)
with a seeded draw; the rest is the training split.

``regrade`` grades recorded episodes again, offline: line 1 of the episode file is the run's meta record, every later
line one episode with its task index and its turns; the last program each episode sent is run against the hidden
tests of the task file given NOW (a repaired suite, a stricter comparator), and the corrected mean score, pass@1 and
pass@n are reported beside the recorded ones. An episode that never sent a program scores 0 in both.

(The roles of halo/entrypoints/code_pool_preparation.py and code_contests_regrade.py, for this package's own code
environment.)"""

from __future__ import annotations

import argparse
import json
import os
import random
import re
import sys
from collections import Counter

_CODE_BLOCK = re.compile(r"```(?:python)?\n(.*?)```", re.DOTALL)
CONSTANT_PROBES = ("", "0", "1", "-1", "YES", "NO", "Yes", "No", "yes", "no", "true", "false")


# ---- shared ----------------------------------------------------------------------------------------------------------
def run_tests(program: str, tests: list[dict], comparator: str = "tokens", sandbox=None, time_limit_s: float = 5.0) -> list[bool]:
    from halo_b200.environments.sandbox import make_sandbox
    from halo_b200.environments.tasks import verdict

    own = sandbox is None
    sandbox = sandbox or make_sandbox("subprocess")
    try:
        out = []
        for t in tests:
            r = sandbox.run(program, t["input"], timeout_s=time_limit_s)
            out.append(r.exit_code == 0 and not r.timed_out and verdict(t["output"], r.stdout, comparator))
        return out
    finally:
        if own:
            sandbox.close()


def read_jsonl(path: str) -> list[dict]:
    return [json.loads(line) for line in open(path) if line.strip()]


# ---- prepare ---------------------------------------------------------------------------------------------------------
def rating_in_bounds(row: dict, lo: float | None, hi: float | None) -> bool:
    if "rating" not in row:
        return True
    r = row["rating"]
    if r is None:
        return lo is None and hi is None          # bounds were asked for: an unrated row cannot be placed
    return (lo is None or r >= lo) and (hi is None or r <= hi)


def load_exclusions(path: str) -> tuple[set, tuple]:
    exact, prefixes = set(), []
    for line in open(path):
        line = line.strip()
        if not line or line.startswith("#"):
            continue
        if line.endswith("*"):
            prefixes.append(line[:-1])
        else:
            exact.add(line)
    return exact, tuple(prefixes)


def excluded(row_id: str, exclusions) -> bool:
    exact, prefixes = exclusions
    return row_id in exact or any(row_id.startswith(p) for p in prefixes)


def suite_accepts_a_constant(row: dict, sandbox=None) -> str | None:
    """The constant answer every hidden test accepts, or None. Probes: a few fixed words and every distinct expected
    output of the suite itself (a suite whose outputs are all the same accepts that one)."""
    from halo_b200.environments.tasks import verdict

    tests = row.get("hidden_tests") or []
    if len(tests) < 2:
        return None                                # one test cannot tell a constant from a program
    comparator = row.get("comparator", "tokens")
    for probe in list(CONSTANT_PROBES) + sorted({t["output"] for t in tests}):
        if all(verdict(t["output"], probe, comparator) for t in tests):
            return probe
    return None


def reference_is_accepted(row: dict, sandbox=None, time_limit_s: float = 5.0) -> bool:
    ref = row.get("reference_solution")
    if not ref:
        return True                                # nothing to check the suite against
    tests = (row.get("public_tests") or []) + (row.get("hidden_tests") or [])
    return all(run_tests(ref, tests, row.get("comparator", "tokens"), sandbox, time_limit_s))


def band_of(rating, width: int, first: int) -> int:
    """Index of the rating band (-1: below the first band or unrated)."""
    if rating is None or rating < first:
        return -1
    return int((rating - first) // width)


def carve_holdout(rows: list[dict], per_band: int, width: int, first: int, seed: int) -> tuple[list[dict], list[dict]]:
    """``(train, test)``: ``per_band`` rows of every band drawn with a seeded shuffle; a band with fewer rows gives them
    all to the hold-out only if it has more than ``per_band`` (a band must keep something to train on)."""
    by_band: dict[int, list[dict]] = {}
    for r in rows:
        by_band.setdefault(band_of(r.get("rating"), width, first), []).append(r)
    train, test = [], []
    for band in sorted(by_band):
        members = sorted(by_band[band], key=lambda r: str(r["id"]))
        random.Random(seed * 1000003 + band).shuffle(members)
        take = per_band if len(members) > per_band else 0
        test += members[:take]
        train += members[take:]
    return train, test


def to_task_row(row: dict) -> dict:
    keep = ("id", "statement", "public_tests", "hidden_tests", "comparator", "rating")
    return {k: row[k] for k in keep if k in row}


def prepare(rows: list[dict], min_rating=None, max_rating=None, exclusions=None, per_band: int = 0, width: int = 400,
            first: int = 800, seed: int = 0, check_suites: bool = True) -> tuple[list[dict], list[dict], Counter]:
    from halo_b200.environments.sandbox import make_sandbox

    drops: Counter = Counter()
    kept = []
    sandbox = make_sandbox("subprocess") if check_suites else None
    try:
        seen = set()
        for row in rows:
            rid = str(row.get("id", ""))
            if not rid or rid in seen:
                drops["no id or duplicate id"] += 1
                continue
            seen.add(rid)
            if not row.get("statement") or not row.get("hidden_tests"):
                drops["no statement or no hidden tests"] += 1
            elif exclusions is not None and excluded(rid, exclusions):
                drops["excluded by the list"] += 1
            elif not rating_in_bounds(row, min_rating, max_rating):
                drops["rating outside the bounds (or unrated)"] += 1
            elif check_suites and suite_accepts_a_constant(row) is not None:
                drops["a constant answer passes every hidden test"] += 1
            elif check_suites and not reference_is_accepted(row, sandbox):
                drops["the reference solution fails its own tests"] += 1
            else:
                kept.append(row)
    finally:
        if sandbox is not None:
            sandbox.close()
    train, test = carve_holdout(kept, per_band, width, first, seed) if per_band > 0 else (kept, [])
    return [to_task_row(r) for r in train], [to_task_row(r) for r in test], drops


# ---- regrade ---------------------------------------------------------------------------------------------------------
def last_program(episode: dict) -> str | None:
    """The last program an episode sent: the last code block of its last assistant turn that holds one."""
    turns = episode.get("turns")
    texts = [t.get("content", "") for t in turns if t.get("role") == "assistant"] if turns else [episode.get("completion", "")]
    for text in reversed(texts):
        found = _CODE_BLOCK.findall(text or "")
        if found:
            return found[-1]
    return None


def regrade(meta: dict, episodes: list[dict], tasks: list[dict], all_or_nothing: bool | None = None) -> tuple[dict, list[dict]]:
    from halo_b200.environments.sandbox import make_sandbox

    if meta.get("env") not in (None, "code"):
        raise ValueError(f"the episodes were recorded in the {meta.get('env')!r} environment; only 'code' episodes re-grade")
    if all_or_nothing is None:
        all_or_nothing = str(meta.get("options", {}).get("all_or_nothing", "")).lower() in ("1", "true", "yes")
    sandbox = make_sandbox("subprocess")
    out = []
    try:
        for ep in episodes:
            ti = ep["task"]
            if not 0 <= ti < len(tasks):
                raise IndexError(f"episode names task {ti}, the task file has {len(tasks)} rows: not the run's selection")
            if "task_id" in ep and "id" in tasks[ti] and str(ep["task_id"]) != str(tasks[ti]["id"]):
                raise ValueError(f"episode of task {ep['task_id']!r} lines up with {tasks[ti]['id']!r} in the task file")
            program = last_program(ep)
            hidden = tasks[ti].get("hidden_tests") or []
            passed = run_tests(program, hidden, tasks[ti].get("comparator", "tokens"), sandbox) if program else [False] * len(hidden)
            frac = sum(passed) / max(1, len(hidden))
            score = float(frac == 1.0) if all_or_nothing else frac
            out.append({**{k: ep[k] for k in ("task", "sample") if k in ep}, "recorded_score": ep.get("score"),
                        "score": score, "hidden_passed": sum(passed), "sent_a_program": program is not None})
    finally:
        sandbox.close()
    n_tasks = len({e["task"] for e in out})
    per_task: dict[int, list[float]] = {}
    for e in out:
        per_task.setdefault(e["task"], []).append(e["score"])
    n = max(len(v) for v in per_task.values()) if per_task else 1
    report = {"episodes": len(out), "tasks": n_tasks,
              "mean_score": sum(e["score"] for e in out) / max(1, len(out)),
              "recorded_mean_score": sum((e["recorded_score"] or 0.0) for e in out) / max(1, len(out)),
              "pass@1": sum(e["score"] >= 1.0 for e in out) / max(1, len(out)),
              f"pass@{n}": sum(any(s >= 1.0 for s in v) for v in per_task.values()) / max(1, n_tasks),
              "changed": sum(1 for e in out if e["recorded_score"] is not None and abs(e["score"] - e["recorded_score"]) > 1e-9)}
    return report, out


def read_episode_file(path: str) -> tuple[dict, list[dict]]:
    rows = read_jsonl(path)
    if rows and "meta" in rows[0]:
        return rows[0]["meta"], rows[1:]
    return {}, rows


# ---- CLI -------------------------------------------------------------------------------------------------------------
def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("prepare")
    p.add_argument("problems")
    p.add_argument("--out-dir", required=True)
    p.add_argument("--min-rating", type=float, default=None)
    p.add_argument("--max-rating", type=float, default=None)
    p.add_argument("--exclude", default="")
    p.add_argument("--holdout-per-band", type=int, default=0)
    p.add_argument("--band-width", type=int, default=400)
    p.add_argument("--first-band", type=int, default=800)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--no-suite-checks", action="store_true")
    r = sub.add_parser("regrade")
    r.add_argument("episodes")
    r.add_argument("--tasks", required=True)
    r.add_argument("--out", default="")
    a = ap.parse_args(argv)
    if a.cmd == "prepare":
        train, test, drops = prepare(read_jsonl(a.problems), a.min_rating, a.max_rating,
                                     load_exclusions(a.exclude) if a.exclude else None, a.holdout_per_band, a.band_width,
                                     a.first_band, a.seed, not a.no_suite_checks)
        os.makedirs(a.out_dir, exist_ok=True)
        for name, rows in (("train", train), ("test", test)):
            with open(os.path.join(a.out_dir, f"{name}.jsonl"), "w") as f:
                for row in rows:
                    f.write(json.dumps(row) + "\n")
        print(json.dumps({"train": len(train), "test": len(test), "dropped": dict(drops)}))
        if not train:
            print("no problem survived the preparation", file=sys.stderr)
            return 1
        return 0
    meta, episodes = read_episode_file(a.episodes)
    report, rows = regrade(meta, episodes, read_jsonl(a.tasks))
    if a.out:
        with open(a.out, "w") as f:
            for row in rows:
                f.write(json.dumps(row) + "\n")
    print(json.dumps(report))
    return 0


if __name__ == "__main__":
    sys.exit(main())
