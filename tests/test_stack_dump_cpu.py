"""All-rank stack dumps from outside: three child processes register the handler and block in two different places; the
tool signals the recorded pids, reads the dumps and names the odd rank out."""

import os
import subprocess
import sys
import time

from halo_b200.diagnostics import stack_dump

_CHILD = """
import sys, time, threading
sys.path.insert(0, {root!r})
from halo_b200.diagnostics import stack_dump
rank = int(sys.argv[1])
stack_dump.install({out!r}, rank)
threading.Thread(target=time.sleep, args=(60,), daemon=True).start()
def waiting_in_the_collective():
    time.sleep(60)
def still_loading_data():
    time.sleep(60)
print("ready", flush=True)
(still_loading_data if rank == 1 else waiting_in_the_collective)()
"""


def test_dump_and_triage(tmp_path):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = str(tmp_path / "run")
    procs = [subprocess.Popen([sys.executable, "-c", _CHILD.format(root=root, out=out), str(r)], stdout=subprocess.PIPE, text=True)
             for r in range(3)]
    try:
        for p in procs:
            assert p.stdout.readline().strip() == "ready"
        time.sleep(0.2)
        recs = stack_dump.recorded_ranks(out)
        assert [r["rank"] for r in recs] == [0, 1, 2] and {r["pid"] for r in recs} == {p.pid for p in procs}
        dumps, problems = stack_dump.dump(out, wait=5.0)
        assert not problems and sorted(dumps) == [0, 1, 2]
        assert stack_dump.where(dumps[0]["main"]).startswith("waiting_in_the_collective")
        assert stack_dump.where(dumps[1]["main"]).startswith("still_loading_data")
        assert dumps[0]["threads"] >= 2
        text = stack_dump.triage(dumps)
        assert "2 rank(s) [0, 2]: waiting_in_the_collective" in text and "the odd one out: rank(s) [1] in still_loading_data" in text
        # a second request appends a second dump; the parser reads the last one
        procs[1].terminate()
        procs[1].wait(timeout=10)
        dumps2, problems2 = stack_dump.dump(out, wait=5.0)
        assert sorted(dumps2) == [0, 2] and any("rank 1" in p and "not running" in p for p in problems2)
        assert stack_dump.main([out, "--wait", "3"]) == 1                     # a missing rank is a non-zero exit
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()


def test_install_is_idempotent(tmp_path):
    a = stack_dump.install(str(tmp_path), 7)
    assert a == stack_dump.install(str(tmp_path), 7) and a.endswith("rank00007.txt")
    assert stack_dump.parse_dump("") == {"main": [], "threads": 0}
    assert stack_dump.dump(str(tmp_path / "nothing"), wait=0.1)[1]
