"""``python -m halo_b200.cli launch <method> <config.yaml> -n N [--key=value ...]`` builds the torchrun
(or plain python) command line for a training method; ``run <tool>`` starts a tool module
(the role of halo/cli.py:1-349). One node by default; ``--nnodes M --node-rank R --rdzv-endpoint host:port`` (or the
``HALO_NNODES`` / ``HALO_NODE_RANK`` / ``HALO_RDZV_ENDPOINT`` variables a cluster launcher exports) starts one node's
share of a multi-node job: the same line on every node, differing only in the node rank."""

from __future__ import annotations

import argparse
import os
import shlex
import subprocess
import sys

METHODS = {
    "sft": "halo_b200.entrypoints.training.sft",
    "dpo": "halo_b200.entrypoints.training.preference",
    "kto": "halo_b200.entrypoints.training.preference",
    "smpo": "halo_b200.entrypoints.training.preference",
    "reward": "halo_b200.entrypoints.training.reward",
    "classification": "halo_b200.entrypoints.training.classification",
    "embedding": "halo_b200.entrypoints.training.embedding",
    "distill": "halo_b200.entrypoints.training.distill",
    "grpo": "halo_b200.entrypoints.training.grpo",
}
TOOLS = {
    "merge-ep-shards": "halo_b200.checkpoint.tools.merge_ep_shards",
    "convert-dtype": "halo_b200.checkpoint.tools.convert_dtype",
    "merge-models": "halo_b200.checkpoint.tools.merge_models",
    "relayout-experts": "halo_b200.checkpoint.tools.relayout_experts",
    "patch-vocab": "halo_b200.checkpoint.tools.patch_vocab",
    "reset-sinks": "halo_b200.checkpoint.tools.reset_sinks",
    "kernel-bench": "benchmarks.kernels",
    "nvlink-health": "halo_b200.diagnostics.nvlink_health",
    "trace-report": "halo_b200.diagnostics.trace_report",
    "stack-dump": "halo_b200.diagnostics.stack_dump",
    "convert-recipe": "halo_b200.configs.convert_recipe",
    "prepare-dataset": "halo_b200.data.preprocessed",
    "deduplicate": "halo_b200.data.deduplication",
    "generate": "halo_b200.entrypoints.generation",
    "evaluate": "halo_b200.entrypoints.evaluation",
    "reward-scoring": "halo_b200.entrypoints.reward_scoring",
    "env-eval": "halo_b200.entrypoints.env_eval",
    "code-tasks": "halo_b200.entrypoints.code_tasks",
    "merge-adapter": "halo_b200.checkpoint.tools.merge_adapter",
    "lowp-convert": "halo_b200.checkpoint.tools.lowp_convert",
    "merge-pp-stages": "halo_b200.checkpoint.tools.merge_pp_stages",
    "reattach-vision": "halo_b200.checkpoint.tools.reattach_vision",
    "weight-push-bench": "benchmarks.weight_push",
    "bench": "bench",
}


def build_command(method: str, config: str, nproc: int, overrides: list[str], port: int = 29500,
                  numa_binding: bool = False, nnodes: int = 1, node_rank: int = 0, rdzv_endpoint: str = "") -> list[str]:
    if method not in METHODS:
        raise SystemExit(f"unknown method {method!r}; choose from {', '.join(sorted(METHODS))}")
    module = METHODS[method]
    extra = [f"--preference_loss={method}"] if method in ("dpo", "kto", "smpo") else []
    if nnodes > 1:
        if not rdzv_endpoint or ":" not in rdzv_endpoint:
            raise SystemExit("a multi-node launch needs --rdzv-endpoint host:port (the first node's address, reachable by all)")
        if not 0 <= node_rank < nnodes:
            raise SystemExit(f"--node-rank {node_rank} is outside 0..{nnodes - 1}")
        host, _, rport = rdzv_endpoint.rpartition(":")
        cmd = [sys.executable, "-m", "torch.distributed.run", f"--nnodes={nnodes}", f"--node-rank={node_rank}",
               f"--nproc-per-node={max(nproc, 1)}", "--master-addr", host, "--master-port", rport]
        if numa_binding:
            cmd += ["--numa-binding", "node"]
        return cmd + ["-m", module, config, *extra, *overrides]
    if nproc <= 1:
        return [sys.executable, "-m", module, config, *extra, *overrides]
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port)]
    if numa_binding:
        cmd += ["--numa-binding", "node"]
    return cmd + ["-m", module, config, *extra, *overrides]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="halo_b200")
    sub = ap.add_subparsers(dest="cmd", required=True)
    la = sub.add_parser("launch")
    la.add_argument("method")
    la.add_argument("config")
    la.add_argument("-n", "--nproc", type=int, default=1)
    la.add_argument("--port", type=int, default=29500)
    la.add_argument("--numa-binding", action="store_true")
    la.add_argument("--dry-run", action="store_true")
    la.add_argument("--nnodes", type=int, default=int(os.environ.get("HALO_NNODES", "1")))
    la.add_argument("--node-rank", type=int, default=int(os.environ.get("HALO_NODE_RANK", "0")))
    la.add_argument("--rdzv-endpoint", default=os.environ.get("HALO_RDZV_ENDPOINT", ""))
    ru = sub.add_parser("run")
    ru.add_argument("tool")
    args, rest = ap.parse_known_args(argv)
    if args.cmd == "launch":
        cmd = build_command(args.method, args.config, args.nproc, rest, args.port, args.numa_binding, args.nnodes,
                            args.node_rank, args.rdzv_endpoint)
    else:
        if args.tool not in TOOLS:
            raise SystemExit(f"unknown tool {args.tool!r}; choose from {', '.join(sorted(TOOLS))}")
        cmd = [sys.executable, "-m", TOOLS[args.tool], *rest]
    if getattr(args, "dry_run", False):
        print(" ".join(shlex.quote(c) for c in cmd))
        return 0
    return subprocess.call(cmd, env=dict(os.environ))


if __name__ == "__main__":
    sys.exit(main())
