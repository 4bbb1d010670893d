"""Score stored completions, or sample-and-keep-the-best:

    python -m halo_b200.entrypoints.reward_scoring score   completions.jsonl --terms terms.yaml --out scored.jsonl
    python -m halo_b200.entrypoints.reward_scoring reject  <checkpoint> --prompts prompts.jsonl --terms terms.yaml \\
                                                            --n 8 --keep 1 --out sft.jsonl

``score`` adds ``reward`` and ``reward_parts`` to every row that has a ``completion`` (and optional ``target``), resuming
from a partially written output. ``reject`` is rejection sampling: ``n`` completions per prompt from the checkpoint, scored
with the same terms, the best ``keep`` (at or above ``--min-reward``) written as prompt / completion rows ready for
supervised fine-tuning. The roles of the reference's offline reward scoring and rejection-sampling CLIs
(halo/entrypoints/{offline_reward_scoring,reward_scoring,rejection_sampling}.py)."""

from __future__ import annotations

import argparse
import json
import os
import sys


def load_terms(path: str):
    import yaml

    from halo_b200.rewards.terms import RewardComposer, parse_terms

    spec = yaml.safe_load(open(path))
    return RewardComposer(parse_terms(spec["reward_terms"] if isinstance(spec, dict) else spec))


def score_file(rows_path: str, composer, out_path: str) -> dict:
    done = 0
    if os.path.isfile(out_path):
        done = sum(1 for line in open(out_path) if line.strip())          # resume: rows are written in order
    rows = [json.loads(line) for line in open(rows_path) if line.strip()]
    total = 0.0
    with open(out_path, "a") as out:
        for row in rows[done:]:
            episode = {"completion": row["completion"], "target": row.get("target", row.get("answer", "")), **row.get("episode", {})}
            row["reward"], row["reward_parts"] = composer.score(episode)
            total += row["reward"]
            out.write(json.dumps(row) + "\n")
            out.flush()
    n = len(rows) - done
    return {"scored": n, "skipped": done, "mean_reward": total / max(n, 1), "scorer_failures": composer.failures}


def reject(checkpoint: str, prompts_path: str, composer, out_path: str, n: int, keep: int, min_reward: float, args) -> dict:
    import torch

    from halo_b200.entrypoints.generation import generate_rows, load_for_inference, read_prompts
    from halo_b200.inference.generate import SamplingParams
    from transformers import AutoTokenizer

    tokenizer = AutoTokenizer.from_pretrained(checkpoint)
    model = load_for_inference(checkpoint, args.device or ("cuda" if torch.cuda.is_available() else "cpu"), args.adapter)
    rows = read_prompts(prompts_path, tokenizer)
    params = SamplingParams(args.max_new_tokens, args.temperature, args.top_k, args.top_p, (), args.seed)
    records = generate_rows(model, rows, params, n, args.batch, tokenizer, tokenizer.eos_token_id)
    by_prompt: dict[int, list] = {}
    for rec in records:
        target = rows[rec["index"]].get("target", rows[rec["index"]].get("answer", ""))
        rec["reward"], rec["reward_parts"] = composer.score({"completion": rec["completion"], "target": target})
        by_prompt.setdefault(rec["index"], []).append(rec)
    kept = 0
    with open(out_path, "w") as out:
        for i in sorted(by_prompt):
            best = sorted(by_prompt[i], key=lambda r: -r["reward"])[:keep]
            for rec in best:
                if rec["reward"] < min_reward:
                    continue
                row = {"prompt": rows[i].get("prompt"), "messages": rows[i].get("messages"), "completion": rec["completion"],
                       "reward": rec["reward"]}
                out.write(json.dumps({k: v for k, v in row.items() if v is not None}) + "\n")
                kept += 1
    return {"prompts": len(by_prompt), "sampled": len(records), "kept": kept}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    s = sub.add_parser("score")
    s.add_argument("rows")
    s.add_argument("--terms", required=True)
    s.add_argument("--out", required=True)
    r = sub.add_parser("reject")
    r.add_argument("checkpoint")
    r.add_argument("--prompts", required=True)
    r.add_argument("--terms", required=True)
    r.add_argument("--out", required=True)
    r.add_argument("--n", type=int, default=8)
    r.add_argument("--keep", type=int, default=1)
    r.add_argument("--min-reward", type=float, default=float("-inf"))
    r.add_argument("--adapter", default="")
    r.add_argument("--device", default="")
    r.add_argument("--batch", type=int, default=32)
    r.add_argument("--max-new-tokens", type=int, default=512)
    r.add_argument("--temperature", type=float, default=1.0)
    r.add_argument("--top-p", type=float, default=1.0)
    r.add_argument("--top-k", type=int, default=0)
    r.add_argument("--seed", type=int, default=0)
    args = ap.parse_args(argv)
    composer = load_terms(args.terms)
    if args.cmd == "score":
        print(json.dumps(score_file(args.rows, composer, args.out)))
    else:
        print(json.dumps(reject(args.checkpoint, args.prompts, composer, args.out, args.n, args.keep, args.min_reward, args)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
