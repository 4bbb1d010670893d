"""Generate from a checkpoint:  python -m halo_b200.entrypoints.generation <checkpoint> --prompts prompts.jsonl --out out.jsonl

Prompts are JSONL rows with ``prompt`` (text, needs the checkpoint's tokenizer), ``messages`` (chat turns, rendered
with the tokenizer's chat template) or ``prompt_ids``; every row is sampled ``--n`` times in batches of ``--batch``
sequences. Output rows carry the prompt, the completion (ids, and text when a tokenizer is there), the summed
log-probability and the finish reason. ``--adapter`` folds low-rank adapters in first. The role of the reference's
generation CLI (halo/entrypoints/generation.py)."""

from __future__ import annotations

import argparse
import json
import sys

import numpy as np
import torch


def load_for_inference(checkpoint: str, device: str, adapter: str = ""):
    from halo_b200.checkpoint.load import from_pretrained

    dev = torch.device(device)
    model = from_pretrained(checkpoint, device=dev, dtype=torch.bfloat16 if dev.type == "cuda" else torch.float32,
                            gradient_checkpointing=False)
    if adapter:
        from halo_b200.peft.lora import apply_lora, load_adapters, merge_adapters_into_weights, read_adapter_spec

        apply_lora(model, read_adapter_spec(adapter))
        load_adapters(model, adapter)
        merge_adapters_into_weights(model)
    return model.eval()


def read_prompts(path: str, tokenizer):
    rows = [json.loads(line) for line in open(path) if line.strip()]
    for r in rows:
        if "prompt_ids" in r:
            continue
        if tokenizer is None:
            raise ValueError("text prompts need a tokenizer beside the checkpoint")
        if "messages" in r:
            from halo_b200.data.chat_render import template_ids

            r["prompt_ids"] = template_ids(tokenizer, r["messages"], True)
        else:
            r["prompt_ids"] = tokenizer(r["prompt"])["input_ids"]
    return rows


def generate_rows(model, rows, params, n: int, batch: int, tokenizer=None, eos_token_id=None):
    from halo_b200.inference.generate import Generator, SamplingParams

    gen = Generator(model, eos_token_id=eos_token_id)
    jobs = [(i, k) for i in range(len(rows)) for k in range(n)]
    out = []
    for lo in range(0, len(jobs), batch):
        chunk = jobs[lo:lo + batch]
        p = SamplingParams(params.max_new_tokens, params.temperature, params.top_k, params.top_p, params.stop_token_ids,
                           None if params.seed is None else params.seed + lo)
        results = gen.generate([np.asarray(rows[i]["prompt_ids"]) for i, _ in chunk], p)
        for (i, k), g in zip(chunk, results):
            rec = {"index": i, "sample": k, "prompt_ids": list(map(int, g.prompt_ids)), "completion_ids": list(map(int, g.token_ids)),
                   "logprob": float(g.logprobs.sum()), "finish_reason": g.finish_reason}
            if tokenizer is not None:
                rec["completion"] = tokenizer.decode(rec["completion_ids"], skip_special_tokens=True)
            for key in ("prompt", "messages", "id"):
                if key in rows[i]:
                    rec[key] = rows[i][key]
            out.append(rec)
    return out


def main(argv=None) -> int:
    from halo_b200.inference.generate import SamplingParams

    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("checkpoint")
    ap.add_argument("--prompts", required=True)
    ap.add_argument("--out", default="-")
    ap.add_argument("--adapter", default="")
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--n", type=int, default=1)
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--max-new-tokens", type=int, default=256)
    ap.add_argument("--temperature", type=float, default=1.0)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--top-k", type=int, default=0)
    ap.add_argument("--seed", type=int, default=0)
    args = ap.parse_args(argv)
    tokenizer = None
    try:
        from transformers import AutoTokenizer

        tokenizer = AutoTokenizer.from_pretrained(args.checkpoint)
    except Exception:  # noqa: BLE001 - a checkpoint without tokenizer files serves token-id prompts
        pass
    model = load_for_inference(args.checkpoint, args.device, args.adapter)
    rows = read_prompts(args.prompts, tokenizer)
    params = SamplingParams(args.max_new_tokens, args.temperature, args.top_k, args.top_p, (), args.seed)
    records = generate_rows(model, rows, params, args.n, args.batch, tokenizer, getattr(tokenizer, "eos_token_id", None))
    sink = sys.stdout if args.out == "-" else open(args.out, "w")
    for rec in records:
        sink.write(json.dumps(rec) + "\n")
    if sink is not sys.stdout:
        sink.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
