"""Orchestrator mechanics that need no GPU: a step's whole process group ends with it, a signal to the
orchestrator ends the running step first, and the knob sweep is never merged into a batched launch."""
import os
import signal
import subprocess
import sys
import time

from tileccl_b200.bench import run_all

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _alive(pid: int) -> bool:
    try:
        os.kill(pid, 0)
    except ProcessLookupError:
        return False
    # a zombie still answers signal 0: look at its state
    try:
        with open(f"/proc/{pid}/stat") as f:
            return f.read().split(")")[-1].split()[0] != "Z"
    except OSError:
        return False


def test_step_time_out_ends_the_whole_process_group(tmp_path):
    pidfile = tmp_path / "child.pid"
    # the step starts a grandchild (as a launcher starts ranks) and both sleep far longer than the limit
    code = ("import subprocess, sys, time; p = subprocess.Popen([sys.executable, '-c', 'import time; time.sleep(600)']); "
            f"open(r'{pidfile}', 'w').write(str(p.pid)); time.sleep(600)")
    logs = []
    t0 = time.time()
    rc = run_all.run_step("sleeper", [sys.executable, "-c", code], 2.0, tmp_path, logs.append)
    assert rc == 124 and time.time() - t0 < 60
    grandchild = int(pidfile.read_text())
    for _ in range(50):
        if not _alive(grandchild):
            break
        time.sleep(0.1)
    assert not _alive(grandchild)
    assert "sleeper rc=124" in (tmp_path / "manifest.txt").read_text()


def test_signal_to_the_orchestrator_ends_the_running_step(tmp_path):
    pidfile = tmp_path / "step.pid"
    driver = (
        "import sys, os\n"
        f"sys.path.insert(0, r'{ROOT}')\n"
        "from pathlib import Path\n"
        "from tileccl_b200.bench import run_all\n"
        "run_all.install_signal_handlers(lambda m: None)\n"
        f"code = \"import os, time; open(r'{pidfile}', 'w').write(str(os.getpid())); time.sleep(600)\"\n"
        f"run_all.run_step('held', [sys.executable, '-c', code], 600.0, Path(r'{tmp_path}'), lambda m: None)\n")
    p = subprocess.Popen([sys.executable, "-c", driver])
    for _ in range(300):
        if pidfile.exists() and pidfile.read_text():
            break
        time.sleep(0.1)
    step_pid = int(pidfile.read_text())
    assert _alive(step_pid)
    p.send_signal(signal.SIGTERM)
    assert p.wait(timeout=60) == 128 + signal.SIGTERM
    for _ in range(50):
        if not _alive(step_pid):
            break
        time.sleep(0.1)
    assert not _alive(step_pid)


def test_tuning_sweep_is_a_launch_of_its_own(tmp_path):
    steps = run_all.plan(8, False, tmp_path, tuning=True)
    merged = run_all.batch_rank_steps(steps, tmp_path)
    names = [s[0] for s in merged]
    assert "tune_fused" in names                                  # not folded into a batch_... step
    batches = [s for s in merged if s[0].startswith("batch_")]
    assert batches and all("tune_fused" not in " ".join(s[1]) for s in batches)
    assert all(limit <= 0.25 * 20000 for _, _, limit, _ in batches)
