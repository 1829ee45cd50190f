"""Native rank launcher: host-side failure detection (no GPU, no device fault).

A rank that raises, exits early or is late is produced on the host; the other ranks must leave
their barrier with an error instead of hanging."""
import subprocess

import pytest

from tileccl_b200 import _build


@pytest.fixture(scope="module")
def selftest():
    outs = _build.build(programs=True)
    return str(outs["launcher_selftest"])


@pytest.mark.parametrize("mode", ["ok", "fail", "exit-early", "slow"])
@pytest.mark.parametrize("world", [2, 4])
def test_launcher_scenarios(selftest, mode, world):
    r = subprocess.run([selftest, "--mode", mode, "--world", str(world), "--timeout", "1.0"], capture_output=True, text=True, timeout=60)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "PASS" in r.stdout


def test_device_probe_runs_in_a_child(selftest):
    r = subprocess.run([selftest, "--probe-devices"], capture_output=True, text=True, timeout=60)
    assert r.returncode == 0 and r.stdout.startswith("devices:")


def test_host_plumbing_selftest(selftest, tmp_path):
    from tileccl_b200 import _build
    exe = str(_build.build(programs=True)["host_selftest"])
    r = subprocess.run([exe, str(tmp_path / "x.csv")], capture_output=True, text=True, timeout=60)
    assert r.returncode == 0 and "PASS" in r.stdout, r.stdout + r.stderr
