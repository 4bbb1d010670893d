"""Evaluate a checkpoint on environment tasks:

    python -m halo_b200.entrypoints.env_eval <checkpoint> --tasks tasks.jsonl --env tool_qa [--n 4] [--option protocol=react]

Every task is played ``--n`` times through the same episode loop training uses (multi-turn, tools, sandboxed code);
the report gives the mean score, pass@1 and pass@n (a task passes when an episode scores 1), the share of episodes
cut for malformed turns or the turn budget, and tool calls per episode. Episodes are written to ``--out`` as JSONL
(line 1 is the run's meta record; ``code_tasks regrade`` grades the recorded programs again offline).
The role of the reference's environment eval runners (halo/entrypoints/{generic_env_eval,code_contests_eval}.py)."""

from __future__ import annotations

import argparse
import asyncio
import json
import sys

import numpy as np
import torch


def evaluate_tasks(model, tokenizer, tasks: list[dict], env_type: str, n: int, sampling, env_options: dict | None = None,
                   composer=None) -> tuple[dict, list[dict]]:
    from halo_b200.environments.episode_loop import play_episode
    from halo_b200.environments.local_policy import LocalPolicy
    from halo_b200.environments.registry import make_environment
    from halo_b200.inference.generate import Generator

    policy = LocalPolicy(Generator(model, eos_token_id=getattr(tokenizer, "eos_token_id", None)), tokenizer, sampling)
    episodes = []

    async def run():
        for ti, task in enumerate(tasks):
            for k in range(n):
                env = make_environment(env_type, task, **(env_options or {}))
                rec = await play_episode(env, policy.for_episode(ti * n + k), composer)
                episodes.append({"task": ti, "sample": k, "score": rec.score, "reward": rec.info.get("reward", rec.score),
                                 "done_reason": rec.done_reason, "tool_calls": rec.tool_calls_used, "n_turns": len(rec.turns),
                                 "completion": rec.completion, "task_id": task.get("id"),
                                 # the policy's turns as the offline re-grader reads them (code_tasks regrade)
                                 "turns": [{"role": "assistant", "content": t.content} for t in rec.turns]})

    with torch.no_grad():
        asyncio.run(run())
    scores = np.array([e["score"] for e in episodes]).reshape(len(tasks), n)
    cut = [e["done_reason"] in ("malformed_turns", "turn_budget", "generation_timeout", "tool_budget") for e in episodes]
    report = {"tasks": len(tasks), "episodes": len(episodes), "mean_score": float(scores.mean()),
              "pass@1": float((scores >= 1.0).mean()), f"pass@{n}": float((scores >= 1.0).any(1).mean()),
              "cut_short": float(np.mean(cut)), "tool_calls_per_episode": float(np.mean([e["tool_calls"] for e in episodes]))}
    return report, episodes


def main(argv=None) -> int:
    from transformers import AutoTokenizer

    from halo_b200.entrypoints.generation import load_for_inference
    from halo_b200.inference.generate import SamplingParams

    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("checkpoint")
    ap.add_argument("--tasks", required=True)
    ap.add_argument("--env", required=True)
    ap.add_argument("--n", type=int, default=1)
    ap.add_argument("--option", action="append", default=[], help="key=value options of the environment")
    ap.add_argument("--adapter", default="")
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--max-new-tokens", type=int, default=512)
    ap.add_argument("--temperature", type=float, default=0.7)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--out", default="")
    args = ap.parse_args(argv)
    tasks = [json.loads(line) for line in open(args.tasks) if line.strip()]
    options = dict(o.split("=", 1) for o in args.option)
    model = load_for_inference(args.checkpoint, args.device, args.adapter)
    tokenizer = AutoTokenizer.from_pretrained(args.checkpoint)
    report, episodes = evaluate_tasks(model, tokenizer, tasks, args.env, args.n,
                                      SamplingParams(args.max_new_tokens, args.temperature, 0, args.top_p), options)
    if args.out:
        with open(args.out, "w") as f:
            # line 1: what the offline re-grader needs to rebuild the run (environment, its options, the task file)
            f.write(json.dumps({"meta": {"env": args.env, "options": options, "tasks": args.tasks, "n": args.n,
                                         "checkpoint": args.checkpoint, "report": report}}) + "\n")
            for e in episodes:
                f.write(json.dumps(e) + "\n")
    print(json.dumps(report))
    return 0


if __name__ == "__main__":
    sys.exit(main())
