"""bench.py prints rank 0's JSON line exactly once: at the normal end, or - when the additional blocks of the line
stall or the launcher ends the job - from the watchdog / the SIGTERM handler, with the blocks that are complete."""

import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r'''
import importlib.util, os, signal, sys, time
spec = importlib.util.spec_from_file_location("bench", os.path.join(sys.argv[1], "bench.py"))
sys.argv = ["bench.py"]
bench = importlib.util.module_from_spec(spec); spec.loader.exec_module(bench)
mode = os.environ["MODE"]
extras = {}
emit = bench._LineEmitter({"value": 1.5}, extras, int(os.environ.get("RANK_UNDER_TEST", "0")))
if mode == "normal":
    emit.arm(30.0); extras["backbone"] = {"ok": 1}; emit.disarm(); emit(); emit()
elif mode == "stall":
    emit.arm(0.3); extras["backbone"] = {"ok": 1}; time.sleep(20); print("NOT-REACHED"); sys.exit(3)
elif mode == "terminated":
    emit.arm(30.0); os.kill(os.getpid(), signal.SIGTERM); time.sleep(20); print("NOT-REACHED"); sys.exit(3)
'''


def _run(mode, rank=0):
    env = dict(os.environ, MODE=mode, RANK_UNDER_TEST=str(rank))
    return subprocess.run([sys.executable, "-c", CHILD, ROOT], env=env, capture_output=True, text=True, timeout=120)


def test_line_is_printed_once_at_the_normal_end():
    proc = _run("normal")
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [l for l in proc.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    assert json.loads(lines[0]) == {"value": 1.5, "backbone": {"ok": 1}}


def test_stalled_blocks_do_not_cost_the_headline():
    proc = _run("stall")
    assert proc.returncode == 0 and "NOT-REACHED" not in proc.stdout, proc.stdout + proc.stderr[-2000:]
    line = json.loads([l for l in proc.stdout.splitlines() if l.startswith("{")][0])
    assert line["value"] == 1.5 and line["backbone"] == {"ok": 1} and "cut short" in line["extras_note"]


def test_a_terminated_job_still_prints_the_line_on_rank_0_only():
    proc = _run("terminated")
    assert proc.returncode == 0 and "NOT-REACHED" not in proc.stdout, proc.stdout + proc.stderr[-2000:]
    assert "terminated" in json.loads(proc.stdout.splitlines()[-1])["extras_note"]
    other = _run("stall", rank=1)  # other ranks leave quietly (a moment after rank 0)
    assert other.returncode == 0 and not [l for l in other.stdout.splitlines() if l.startswith("{")]
