"""Hold a benchmark result to its stored band.

    python bench.py --gpus 1 | python benchmarks/band.py moe30b_ep1_n1
    python benchmarks/band.py --list

A band (``benchmarks/baselines/<name>.json``) stores the command, the measured tokens/s/GPU and peak memory with
their provenance, and tolerances. The check reads the benchmark's JSON line from standard input (or ``--result``),
refuses a result for another model or GPU count, and fails when throughput fell below the band or peak memory grew
beyond it; a result above the band passes and says that the band may be raised. The role of the reference's golden
performance band (tests/common/equivalence/bench_band.py)."""

from __future__ import annotations

import argparse
import json
import os
import sys

HERE = os.path.join(os.path.dirname(os.path.abspath(__file__)), "baselines")


def load_band(name: str) -> dict:
    path = os.path.join(HERE, name + ".json")
    if not os.path.isfile(path):
        raise FileNotFoundError(f"no band named {name!r}; known: {sorted(f[:-5] for f in os.listdir(HERE) if f.endswith('.json'))}")
    return json.load(open(path))


def check(band: dict, result: dict) -> tuple[bool, list[str]]:
    notes, ok = [], True
    if result.get("n_gpus") != band["n_gpus"] or result.get("config", {}).get("model") != band["model"]:
        return False, [f"the result is for {result.get('config', {}).get('model')} on {result.get('n_gpus')} GPUs, the band for "
                       f"{band['model']} on {band['n_gpus']}"]
    per_gpu = result["value"] / result["n_gpus"]
    want, rel = band["tokens_per_s_per_gpu"], band["tolerance"]["tokens_per_s_per_gpu_rel"]
    if per_gpu < want * (1 - rel):
        ok = False
        notes.append(f"throughput {per_gpu:,.0f} tokens/s/GPU is below the band {want:,.0f} -{rel:.0%}")
    elif per_gpu > want * (1 + rel):
        notes.append(f"throughput {per_gpu:,.0f} tokens/s/GPU is above the band {want:,.0f} +{rel:.0%}: raise the band")
    else:
        notes.append(f"throughput {per_gpu:,.0f} tokens/s/GPU is inside the band {want:,.0f} +-{rel:.0%}")
    peak = result.get("config", {}).get("peak_gib", result.get("peak_gib"))
    if band.get("peak_gib") is not None and peak is not None:
        slack = band["tolerance"]["peak_gib_abs"]
        if peak > band["peak_gib"] + slack:
            ok = False
            notes.append(f"peak memory {peak:.1f} GiB is above the band {band['peak_gib']:.1f} +{slack:.0f}")
        else:
            notes.append(f"peak memory {peak:.1f} GiB is inside the band ({band['peak_gib']:.1f} +{slack:.0f})")
    reasons = [r for r in (result.get("clocks") or {}).get("reasons", []) if "thermal" in r or r == "hw_slowdown"]
    if reasons:
        ok = False
        notes.append(f"the run was throttled ({', '.join(reasons)}): measure again")
    return ok, notes


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("band", nargs="?")
    ap.add_argument("--result", default="-", help="file holding the benchmark's JSON line (default: standard input)")
    ap.add_argument("--list", action="store_true")
    args = ap.parse_args(argv)
    if args.list or not args.band:
        for f in sorted(os.listdir(HERE)):
            if f.endswith(".json"):
                b = json.load(open(os.path.join(HERE, f)))
                print(f"{b['name']:18s} {b['tokens_per_s_per_gpu']:>9,.0f} tok/s/GPU  {b['command']}")
        return 0
    text = sys.stdin.read() if args.result == "-" else open(args.result).read()
    lines = [line for line in text.splitlines() if line.strip().startswith("{")]
    if not lines:
        print("no JSON line in the result")
        return 2
    ok, notes = check(load_band(args.band), json.loads(lines[-1]))
    for n in notes:
        print(("ok   " if ok else "FAIL ") + n)
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
