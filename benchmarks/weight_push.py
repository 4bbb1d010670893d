"""Trainer -> rollout weight copy of the 30B-A3B shape on one 8-GPU box: ranks 0..3 train with the experts sharded
four ways (each holds 32 of the 128 experts of every layer and a copy of the replicated tensors), ranks 4..7 each
receive a FULL bf16 copy (about 61 GB) into a resident arena.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 benchmarks/weight_push.py [out.json]

Every trainer stores what it holds straight into the four rollout GPUs (peer stores from one kernel per tensor, no
gather, no collective library call). Timing: CUDA events around the push on every rank, barrier before, MAX over ranks,
median of the timed pushes. The floor is what one rollout GPU must take in: model bytes / link bandwidth per direction.
`--layers N` shrinks the model for a smoke run (the JSON says so).
"""

from __future__ import annotations

import json
import os
import statistics
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

LINK_GBS = 900.0
MEASURED_COPY_GBS = 770.0


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    from halo_b200.models.config import PRESETS
    from halo_b200.ops import _lib
    from halo_b200.weight_sync.group import ShardedCopySync

    args = [a for a in sys.argv[1:] if not a.startswith("--")]
    layers = next((int(a.split("=", 1)[1]) for a in sys.argv[1:] if a.startswith("--layers=")), 0)
    cfg = PRESETS["moe-30b-a3b"]()
    if layers:
        cfg.num_hidden_layers = layers
    n_train = world // 2
    trainers, rollouts = list(range(n_train)), list(range(n_train, world))
    E, H, F, V, L = cfg.num_experts, cfg.hidden_size, cfg.moe_intermediate_size, cfg.vocab_size, cfg.num_hidden_layers
    qkv = (cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * cfg.head_dim
    manifest, replicated = [], []
    for name, shape in (("embed_tokens", (V, H)), ("lm_head", (V, H)), ("norm", (H,))):
        manifest.append((name, shape, torch.bfloat16))
        replicated.append(name)
    for i in range(L):
        for name, shape in ((f"layers.{i}.qkv", (qkv, H)), (f"layers.{i}.o", (H, cfg.num_attention_heads * cfg.head_dim)),
                            (f"layers.{i}.router", (E, H)), (f"layers.{i}.norms", (4, H))):
            manifest.append((name, shape, torch.bfloat16))
            replicated.append(name)
        manifest.append((f"layers.{i}.experts_gate_up", (E, 2 * F, H), torch.bfloat16))
        manifest.append((f"layers.{i}.experts_down", (E, H, F), torch.bfloat16))
    sync = ShardedCopySync(dist.group.WORLD, dev, manifest, trainers, rollouts)
    shapes = {n: s for n, s, _ in manifest}
    pieces = []
    if rank in trainers:
        t = trainers.index(rank)
        e_loc = E // n_train
        g = torch.Generator(device=dev).manual_seed(1234)            # the same values on every trainer: checks are easy
        for k, name in enumerate(replicated):
            if sync.owner_of_replicated(k) == t:
                pieces.append((name, torch.full(shapes[name], float(k % 7 + 1), device=dev, dtype=torch.bfloat16), 0))
        for i in range(L):
            for name in (f"layers.{i}.experts_gate_up", f"layers.{i}.experts_down"):
                full_shape = shapes[name]
                pieces.append((name, torch.full((e_loc,) + tuple(full_shape[1:]), float(t + 1), device=dev, dtype=torch.bfloat16),
                               t * e_loc))
        del g
    times = []
    for it in range(4):
        dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        sync.push(pieces)
        b.record()
        torch.cuda.synchronize()
        ms = torch.tensor([a.elapsed_time(b)], device=dev)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        if it > 0:
            times.append(float(ms.item()))
    ok = torch.ones(1, device=dev)
    if rank in rollouts:
        e_loc = E // n_train
        last = f"layers.{L - 1}.experts_down"
        bank = sync.view(last, shapes[last], torch.bfloat16)
        for t in range(n_train):
            if not bool((bank[t * e_loc:(t + 1) * e_loc] == float(t + 1)).all()):
                ok.zero_()
        k = replicated.index("norm")
        if not bool((sync.view("norm", shapes["norm"], torch.bfloat16) == float(k % 7 + 1)).all()):
            ok.zero_()
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    _lib.raise_on_status(dev)
    if rank == 0:
        total = sync.total
        ms = statistics.median(times)
        rec = {"case": f"weight push {n_train} trainers -> {len(rollouts)} rollout GPUs, full bf16 copy each", "model_bytes": total,
               "layers": L, "reduced": bool(layers), "ms": round(ms, 2), "gb_s_into_each_rollout_gpu": round(total / ms / 1e6, 1),
               "floor_ms_at_900": round(total / (LINK_GBS * 1e6), 2), "floor_ms_at_measured_copy": round(total / (MEASURED_COPY_GBS * 1e6), 2),
               "fraction_of_floor_900": round(total / (LINK_GBS * 1e6) / ms, 3), "payload_verified": bool(ok.item())}
        print(json.dumps(rec), flush=True)
        if args:
            os.makedirs(os.path.dirname(args[0]) or ".", exist_ok=True)
            json.dump(rec, open(args[0], "w"), indent=1)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
