"""All-rank Python stack dumps of a RUNNING (or hung) job, from outside, with no profiler installed.

Every rank registers a handler for ``SIGUSR1`` at start-up that writes all of its threads' stacks to
``<output_dir>/stacks/rank<r>.txt`` (``faulthandler``: it runs in the signal handler itself, so it works while the main
thread is blocked inside a collective) and leaves a small ``rank<r>.json`` with its pid and host. The tool

    python -m halo_b200.diagnostics.stack_dump <output_dir> [--wait 1.0]

signals exactly the recorded pids of this host, waits for the dumps and prints the triage a hang needs: ranks grouped
by where their main thread stands. One hung collective shows as N-1 ranks inside the collective and one rank elsewhere.
Needs no flag at launch beyond the handler every entry point installs, and no py-spy.
(The role of halo/diagnostics/py_spy.py and the reference's py-spy attach script, ``dump`` mode.)"""

from __future__ import annotations

import argparse
import faulthandler
import json
import os
import signal
import socket
import sys
import time

_installed: dict = {}


def _dir(output_dir: str) -> str:
    return os.path.join(output_dir, "stacks")


def install(output_dir: str, rank: int | None = None) -> str | None:
    """Register this process's dump handler (idempotent per directory); returns the dump file's path."""
    if not hasattr(signal, "SIGUSR1"):
        return None
    if rank is None:
        from halo_b200.runtime import ranks

        rank = ranks.get_global_rank()
    d = _dir(output_dir)
    key = (d, rank)
    if key in _installed:
        return _installed[key][0]
    os.makedirs(d, exist_ok=True)
    path = os.path.join(d, f"rank{rank:05d}.txt")
    f = open(path, "a")                                   # kept open: the handler may only write to an open descriptor
    faulthandler.register(signal.SIGUSR1, file=f, all_threads=True, chain=False)
    with open(os.path.join(d, f"rank{rank:05d}.json"), "w") as meta:
        json.dump({"rank": rank, "pid": os.getpid(), "host": socket.gethostname(), "started": time.time()}, meta)
    _installed[key] = (path, f)
    return path


def recorded_ranks(output_dir: str, host: str | None = None) -> list[dict]:
    d, out = _dir(output_dir), []
    if not os.path.isdir(d):
        return out
    for name in sorted(os.listdir(d)):
        if name.endswith(".json"):
            rec = json.load(open(os.path.join(d, name)))
            if host is None or rec.get("host") == host:
                out.append(rec)
    return out


def _alive(pid: int) -> bool:
    try:
        os.kill(pid, 0)
        return True
    except OSError:
        return False


def parse_dump(text: str) -> dict:
    """The LAST dump in a rank's file: ``{"main": [frames innermost first], "threads": n}``; a frame is
    ``function (file:line)``. The thread the signal handler ran on - the main thread - is the one the dump marks
    ``Current thread``."""
    stanzas, cur = [], None
    for line in text.splitlines():
        if line.startswith(("Thread 0x", "Current thread 0x")):
            cur = {"current": line.startswith("Current"), "frames": []}
            stanzas.append(cur)
        elif line.startswith("  File ") and cur is not None:
            try:                                             # '  File "path", line N in func'
                path = line.split('"')[1]
                lineno = line.split(", line ")[1].split(" ")[0]
                func = line.rsplit(" in ", 1)[1]
                cur["frames"].append(f"{func} ({os.path.basename(path)}:{lineno})")
            except IndexError:
                cur["frames"].append(line.strip())
    currents = [i for i, st in enumerate(stanzas) if st["current"]]
    if not currents:
        return {"main": [], "threads": 0}
    return {"main": stanzas[currents[-1]]["frames"], "threads": max(1, len(stanzas) // len(currents))}


def where(frames: list[str]) -> str:
    """The frame that names where a rank stands: the innermost frame outside the standard library's waiting helpers."""
    skip = ("threading.py", "selectors.py", "queue.py", "socket.py", "connection.py", "popen_fork.py")
    for fr in frames:
        if not any(s in fr for s in skip):
            return fr
    return frames[0] if frames else "(no Python frames)"


def triage(per_rank: dict[int, dict]) -> str:
    groups: dict[str, list[int]] = {}
    for r, d in sorted(per_rank.items()):
        groups.setdefault(where(d["main"]), []).append(r)
    lines = [f"{len(per_rank)} rank(s) dumped; main threads stand in {len(groups)} place(s):"]
    for place, rs in sorted(groups.items(), key=lambda kv: (-len(kv[1]), kv[0])):
        lines.append(f"  {len(rs):3d} rank(s) {rs if len(rs) <= 16 else str(rs[:16])[:-1] + ', ...]'}: {place}")
    if len(groups) > 1:
        odd = min(groups.items(), key=lambda kv: len(kv[1]))
        lines.append(f"the odd one out: rank(s) {odd[1]} in {odd[0]} - a collective the others wait in cannot finish without them")
    return "\n".join(lines)


def dump(output_dir: str, wait: float = 1.0, host: str | None = None) -> tuple[dict[int, dict], list[str]]:
    """Signal this host's recorded ranks and read their dumps back. Returns ``({rank: parsed dump}, problems)``."""
    host = host or socket.gethostname()
    recs, problems, sizes = recorded_ranks(output_dir, host), [], {}
    if not recs:
        problems.append(f"no rank of host {host!r} has registered under {_dir(output_dir)!r}")
    for rec in recs:
        path = os.path.join(_dir(output_dir), f"rank{rec['rank']:05d}.txt")
        sizes[rec["rank"]] = os.path.getsize(path) if os.path.isfile(path) else 0
        if not _alive(rec["pid"]):
            problems.append(f"rank {rec['rank']} (pid {rec['pid']}) is not running")
            continue
        os.kill(rec["pid"], signal.SIGUSR1)               # the exact pid the rank recorded, nothing matched by name
    deadline = time.monotonic() + max(wait, 0.1)
    out: dict[int, dict] = {}
    while time.monotonic() < deadline and len(out) + len(problems) < len(recs):
        time.sleep(0.05)
        for rec in recs:
            r = rec["rank"]
            path = os.path.join(_dir(output_dir), f"rank{r:05d}.txt")
            if r not in out and os.path.isfile(path) and os.path.getsize(path) > sizes[r]:
                text = open(path).read()
                if "Current thread" in text[sizes[r]:] or "Thread 0x" in text[sizes[r]:]:
                    out[r] = parse_dump(text)
    for rec in recs:
        if rec["rank"] not in out and _alive(rec["pid"]):
            problems.append(f"rank {rec['rank']} (pid {rec['pid']}) wrote no dump within {wait} s")
    return out, problems


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("output_dir")
    ap.add_argument("--wait", type=float, default=1.0, help="seconds to wait for the dumps")
    ap.add_argument("--full", action="store_true", help="print every rank's main-thread stack, not only the triage")
    a = ap.parse_args(argv)
    dumps, problems = dump(a.output_dir, a.wait)
    if dumps:
        print(triage(dumps))
        if a.full:
            for r, d in sorted(dumps.items()):
                print(f"--- rank {r} ({d['threads']} threads), innermost first")
                for fr in d["main"]:
                    print("   ", fr)
    for p in problems:
        print("problem:", p, file=sys.stderr)
    return 1 if problems else 0


if __name__ == "__main__":
    sys.exit(main())
