"""Score a checkpoint on held-out text:  python -m halo_b200.entrypoints.evaluation <checkpoint> --data eval.jsonl

Reports the mean next-token loss and perplexity over packed rows (``{"input_ids": [...]}`` or ``{"text": "..."}``
rows; with ``--completion-only`` and ``prompt`` / ``completion`` fields only completion tokens count), and with
``--mtp`` the multi-token-prediction head's loss and draft acceptance. The role of the reference's evaluation CLI
(halo/entrypoints/, halo/trainers/loop/evaluation.py)."""

from __future__ import annotations

import argparse
import json
import math
import sys

import numpy as np
import torch


@torch.no_grad()
def evaluate_rows(model, docs: list, row_length: int = 8192, masks: list | None = None, mtp: bool = False) -> dict:
    from halo_b200.data.packing import pack_documents

    dev = next(model.parameters()).device
    total, count = 0.0, 0
    accepted = scored = 0
    head_total = 0.0
    rows, cur, cur_len = [], [], 0
    for i, d in enumerate(docs):
        d = np.asarray(d)[:row_length]
        if cur and cur_len + len(d) > row_length:
            rows.append(cur)
            cur, cur_len = [], 0
        cur.append(i)
        cur_len += len(d)
    if cur:
        rows.append(cur)
    for idx in rows:
        b = pack_documents([np.asarray(docs[i])[:row_length] for i in idx],
                           label_masks=None if masks is None else [np.asarray(masks[i], dtype=bool)[:row_length] for i in idx]).to(dev)
        n = int((b.labels != -100).sum())
        if n == 0:
            continue
        ctx = model.make_context(b.position_ids.reshape(-1), b.cu_seqlens)
        logp, _ = model.token_logprobs(b.input_ids, b.position_ids, b.cu_seqlens, b.labels, ctx=ctx)
        total += float(-(logp * (b.labels.reshape(-1) != -100)).sum())
        count += n
        if mtp and model.mtp is not None:
            from halo_b200.models.mtp import draft_acceptance, shifted_targets
            from halo_b200.ops.cross_entropy import linear_logprobs

            ctx = model.make_context(b.position_ids.reshape(-1), b.cu_seqlens)
            states = model.mtp_states(model.trunk_states(b.input_ids, ctx), b.input_ids, ctx)
            targets = shifted_targets(b.labels, b.cu_seqlens)
            a, s = draft_acceptance(states, model.head_weight(), targets)
            lp, _ = linear_logprobs(states, model.head_weight(), targets)
            head_total += float(-(lp * (targets != -100)).sum())
            accepted, scored = accepted + int(a), scored + int(s)
    loss = total / max(count, 1)
    out = {"loss": loss, "perplexity": math.exp(min(loss, 50.0)), "tokens": count, "rows": len(rows)}
    if mtp and scored:
        out.update({"mtp_loss": head_total / scored, "mtp_acceptance": accepted / scored})
    return out


def main(argv=None) -> int:
    from halo_b200.entrypoints.generation import load_for_inference

    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("checkpoint")
    ap.add_argument("--data", required=True)
    ap.add_argument("--adapter", default="")
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--row-length", type=int, default=8192)
    ap.add_argument("--completion-only", action="store_true")
    ap.add_argument("--mtp", action="store_true")
    args = ap.parse_args(argv)
    rows = [json.loads(line) for line in open(args.data) if line.strip()]
    tokenizer = None
    if rows and "input_ids" not in rows[0]:
        from transformers import AutoTokenizer

        tokenizer = AutoTokenizer.from_pretrained(args.checkpoint)
    docs, masks = [], ([] if args.completion_only else None)
    for r in rows:
        if "input_ids" in r:
            docs.append(r["input_ids"])
            if masks is not None:
                masks.append(r.get("loss_mask") or [1] * len(r["input_ids"]))
        elif "prompt" in r and "completion" in r:
            p, c = tokenizer(r["prompt"])["input_ids"], tokenizer(r["completion"], add_special_tokens=False)["input_ids"]
            docs.append(p + c)
            if masks is not None:
                masks.append([0] * len(p) + [1] * len(c))
        else:
            ids = tokenizer(r["text"])["input_ids"]
            docs.append(ids)
            if masks is not None:
                masks.append([1] * len(ids))
    model = load_for_inference(args.checkpoint, args.device, args.adapter)
    print(json.dumps(evaluate_rows(model, docs, args.row_length, masks, args.mtp)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
