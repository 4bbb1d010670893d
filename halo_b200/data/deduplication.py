"""Near-duplicate removal for a text corpus: every row becomes a unit vector, and a row is dropped when its cosine
similarity to a row that is already kept reaches the threshold.

    python -m halo_b200.data.deduplication in.jsonl out.jsonl --field text --threshold 0.9 [--model DIR] [--device cuda]

Vectors come from hashed character n-grams by default (no model needed: catches copies that differ in whitespace,
casing, a few edited words) or, with ``--model``, from the mean of a decoder's final hidden states over the row's
tokens (semantic duplicates). The search is exact and blocked: a block of rows is compared with everything kept so
far in one matrix product, then resolved inside the block in order, so the result does not depend on the block size
and equals the greedy pass over the rows one by one. Rows are visited in a seeded order, which decides which
member of a duplicate group survives; the output keeps the input order.
(The role of halo/data/deduplication.py and scripts/before_training/deduplicate_dataset.py, with the similarity
search as plain matrix products instead of a FAISS index.)"""

from __future__ import annotations

import argparse
import json
import zlib

import numpy as np
import torch

SHUFFLE_SEED = 42


def ngram_vectors(texts, n: int = 5, dim: int = 4096, lowercase: bool = True) -> torch.Tensor:
    """Unit vectors ``[N, dim]`` of hashed character ``n``-gram counts (whitespace runs collapsed)."""
    out = np.zeros((len(texts), dim), dtype=np.float32)
    for i, text in enumerate(texts):
        t = " ".join(str(text).split())
        t = t.lower() if lowercase else t
        data = t.encode("utf-8")
        if len(data) < n:
            data = data + b" " * (n - len(data))
        for j in range(len(data) - n + 1):
            out[i, zlib.crc32(data[j:j + n]) % dim] += 1.0
    v = torch.from_numpy(out)
    return v / v.norm(dim=1, keepdim=True).clamp_min(1e-12)


@torch.no_grad()
def model_vectors(texts, model, tokenizer, max_tokens: int = 512, rows_per_pass: int = 32) -> torch.Tensor:
    """Unit vectors from the mean of the decoder's final hidden states over each row's tokens; rows are packed into
    one varlen sequence per pass (no padding)."""
    from halo_b200.data.packing import pack_documents

    device = next(model.parameters()).device
    out = []
    for lo in range(0, len(texts), rows_per_pass):
        docs = [np.asarray(tokenizer(str(t), add_special_tokens=False)["input_ids"][:max_tokens] or [0]) for t in texts[lo:lo + rows_per_pass]]
        b = pack_documents(docs).to(device)
        h = model.hidden_states(b.input_ids, b.position_ids, b.cu_seqlens).float()
        cu = [int(x) for x in b.cu_seqlens]
        out.append(torch.stack([h[a:z].mean(0) for a, z in zip(cu[:-1], cu[1:])][:len(docs)]).cpu())
    v = torch.cat(out)
    return v / v.norm(dim=1, keepdim=True).clamp_min(1e-12)


@torch.no_grad()
def keep_mask(vectors: torch.Tensor, threshold: float, block: int = 4096, seed: int | None = SHUFFLE_SEED, device=None) -> np.ndarray:
    """``True`` for the rows that survive. ``vectors [N, D]`` must be unit rows."""
    n = vectors.shape[0]
    order = np.random.default_rng(seed).permutation(n) if seed is not None else np.arange(n)
    v = vectors[torch.from_numpy(order)].to(device or vectors.device)
    kept_rows: list[torch.Tensor] = []
    kept = np.zeros(n, dtype=bool)
    for lo in range(0, n, block):
        blk = v[lo:lo + block]
        dup = torch.zeros(blk.shape[0], dtype=torch.bool, device=blk.device)
        for prior in kept_rows:                              # against everything kept in earlier blocks
            dup |= (blk @ prior.t()).amax(dim=1) >= threshold
        inside = (blk @ blk.t()) >= threshold                # inside the block: in order, against kept earlier rows only
        alive = (~dup).cpu().numpy()
        inside = inside.cpu().numpy()
        for i in range(blk.shape[0]):
            if alive[i] and i and (inside[i, :i] & alive[:i]).any():
                alive[i] = False
        kept[lo:lo + blk.shape[0]] = alive
        if alive.any():
            kept_rows.append(blk[torch.from_numpy(alive).to(blk.device)])
    out = np.zeros(n, dtype=bool)
    out[order] = kept
    return out


def deduplicate_texts(texts, threshold: float = 0.9, vectors: torch.Tensor | None = None, **kw) -> np.ndarray:
    return keep_mask(ngram_vectors(texts) if vectors is None else vectors, threshold, **kw)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("source")
    ap.add_argument("destination")
    ap.add_argument("--field", default="text")
    ap.add_argument("--threshold", type=float, default=0.9)
    ap.add_argument("--model", default="", help="checkpoint directory: semantic vectors instead of hashed n-grams")
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--block", type=int, default=4096)
    args = ap.parse_args(argv)
    rows = [json.loads(line) for line in open(args.source) if line.strip()]

    def text_of(row):
        value = row[args.field]
        if isinstance(value, list):                          # a conversation: its turns joined
            return "\n".join(str(m.get("content", "")) if isinstance(m, dict) else str(m) for m in value)
        return str(value)

    texts = [text_of(r) for r in rows]
    if args.model:
        from transformers import AutoTokenizer

        from halo_b200.checkpoint.load import from_pretrained

        model = from_pretrained(args.model, device=args.device, gradient_checkpointing=False)
        vectors = model_vectors(texts, model, AutoTokenizer.from_pretrained(args.model))
    else:
        vectors = ngram_vectors(texts)
    keep = keep_mask(vectors, args.threshold, block=args.block, device=args.device)
    with open(args.destination, "w") as f:
        for row, k in zip(rows, keep):
            if k:
                f.write(json.dumps(row, ensure_ascii=False) + "\n")
    print(json.dumps({"rows": len(rows), "kept": int(keep.sum()), "dropped": int((~keep).sum()), "threshold": args.threshold}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
