"""Tensor records for before / after comparisons of a change that must not alter numerics.

    python benchmarks/records.py record out.json            # run the fixed workloads at this commit
    python benchmarks/records.py compare base.json head.json [--tolerance 0]

``record`` runs small deterministic workloads on CPU - a tiny MoE for three optimizer steps in one process, and the same
under expert parallelism on two gloo ranks - and stores, per step, the loss and a digest plus the norm of every
parameter's gradient and of the updated weights. ``compare`` holds two such files against each other: bit-for-bit by
default (digests), or within a relative tolerance on the norms. Run it at a base commit and at the change (for instance
in two worktrees): a refactor that "only moved code" compares equal. The role of the reference's equivalence gates
against a base commit (tests/common/equivalence/{ep_bitwise,tensor_records}.py)."""

from __future__ import annotations

import argparse
import hashlib
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def digest(t: torch.Tensor) -> str:
    return hashlib.blake2b(t.detach().contiguous().cpu().numpy().tobytes(), digest_size=12).hexdigest()


def _workload(rank: int, world: int, out_path: str):
    import torch.distributed as dist

    from halo_b200.data.packing import synthetic_packed_batch
    from halo_b200.models.config import tiny_moe_config
    from halo_b200.models.qwen3 import build_model
    from halo_b200.trainers.engine import TrainEngine

    torch.manual_seed(0)
    cfg = tiny_moe_config()
    transport = parallel = None
    if world > 1:
        from halo_b200.parallel.expert_parallel import CollectiveTransport
        from halo_b200.parallel.runtime import ParallelRuntime

        transport = CollectiveTransport(dist.group.WORLD)
        parallel = ParallelRuntime("cpu", dp_group=dist.group.WORLD, ep_group=dist.group.WORLD, transport=transport)
    model = build_model(cfg, device="cpu", seed=0, transport=transport)
    engine = TrainEngine(model, torch.optim.AdamW(model.parameters(), lr=1e-3), "cpu", parallel=parallel)
    steps = []
    for step in range(3):
        batch = synthetic_packed_batch(256, cfg.vocab_size, seed=10 * step + rank, lo=16, hi=96)
        grads = {}
        hooks = [p.register_hook(lambda g, n=n: grads.__setitem__(n, (digest(g), float(g.float().norm())))) for n, p in model.named_parameters()]
        out = engine.train_step(batch)
        for h in hooks:
            h.remove()
        steps.append({"loss": float(out.loss.reshape(-1)[0]), "grad_norm": float(out.grad_norm),
                      "grads": grads, "weights": {n: (digest(p), float(p.detach().float().norm())) for n, p in model.named_parameters()}})
    if world == 1:
        return steps
    gathered = [None] * world
    dist.all_gather_object(gathered, steps)
    if rank == 0:
        json.dump(gathered, open(out_path, "w"))
    return None


def record(path: str) -> None:
    import tempfile

    from tests.common.gloo import run_gloo_ranks

    single = _workload(0, 1, "")
    with tempfile.TemporaryDirectory() as d:
        ep_path = os.path.join(d, "ep.json")
        run_gloo_ranks(_workload, 2, args=(ep_path,), timeout=300.0)
        ep = json.load(open(ep_path))
    json.dump({"torch": torch.__version__, "workloads": {"single": [single], "ep2": ep}}, open(path, "w"), indent=1)


def compare(a: dict, b: dict, tolerance: float = 0.0) -> list[str]:
    diffs = []
    for name in sorted(set(a["workloads"]) | set(b["workloads"])):
        wa, wb = a["workloads"].get(name), b["workloads"].get(name)
        if wa is None or wb is None:
            diffs.append(f"{name}: present in one record only")
            continue
        for rank, (ra, rb) in enumerate(zip(wa, wb)):
            for step, (sa, sb) in enumerate(zip(ra, rb)):
                where = f"{name} rank {rank} step {step}"
                if tolerance == 0.0 and sa["loss"] != sb["loss"] or abs(sa["loss"] - sb["loss"]) > tolerance * max(1.0, abs(sa["loss"])):
                    diffs.append(f"{where}: loss {sa['loss']!r} vs {sb['loss']!r}")
                for kind in ("grads", "weights"):
                    for key in sorted(set(sa[kind]) | set(sb[kind])):
                        va, vb = sa[kind].get(key), sb[kind].get(key)
                        if va is None or vb is None:
                            diffs.append(f"{where}: {kind[:-1]} of {key} present in one record only")
                        elif tolerance == 0.0 and va[0] != vb[0]:
                            diffs.append(f"{where}: {kind[:-1]} of {key} differs bit-wise (norms {va[1]:.6g} vs {vb[1]:.6g})")
                        elif tolerance > 0.0 and abs(va[1] - vb[1]) > tolerance * max(abs(va[1]), 1e-12):
                            diffs.append(f"{where}: {kind[:-1]} norm of {key} {va[1]:.6g} vs {vb[1]:.6g}")
    return diffs


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    r = sub.add_parser("record")
    r.add_argument("out")
    c = sub.add_parser("compare")
    c.add_argument("base")
    c.add_argument("head")
    c.add_argument("--tolerance", type=float, default=0.0)
    args = ap.parse_args(argv)
    if args.cmd == "record":
        record(args.out)
        print(f"recorded to {args.out}")
        return 0
    diffs = compare(json.load(open(args.base)), json.load(open(args.head)), args.tolerance)
    for d in diffs[:40]:
        print(d)
    print(f"{len(diffs)} differences" if diffs else "the records are equal")
    return 1 if diffs else 0


if __name__ == "__main__":
    sys.exit(main())
