"""Fused ops across real GPUs (2, 4, 8 where present): one process per GPU."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]

HERE = os.path.dirname(os.path.abspath(__file__))


def _run(world: int, port: int):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "_mp_worker.py")]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    return subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_fused_ops_multi_gpu(native_lib, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    r = _run(world, 29600 + world)
    assert r.returncode == 0 and "WORKER_OK" in r.stdout, r.stdout[-4000:] + r.stderr[-4000:]


def test_native_launcher_driver_two_gpus(native_lib):
    """The C++ driver: ranks forked by the native launcher, cudaIpc exchange through its shared blob."""
    from tileccl_b200 import _build
    exe = str(_build.build(programs=True)["exp3_gemm_rs_fused"])
    r = subprocess.run([exe, "--ndev", "2", "--m", "2048", "--n", "1024", "--k", "512", "--iters", "5", "--warmup", "2", "--verify"],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "FAIL" not in r.stdout and "max over ranks" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


def test_native_exp2_and_epilogue_drivers_two_gpus(native_lib):
    from tileccl_b200 import _build
    outs = _build.build(programs=True)
    r = subprocess.run([str(outs["exp2_ag_gemm_granularity"]), "--ndev", "2", "--m", "2048", "--k", "512", "--n", "512", "--gather-rows", "256,1024",
                        "--iters", "3", "--warmup", "1", "--verify"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "FAIL" not in r.stdout and r.stdout.count(" ok") == 2, r.stdout[-3000:] + r.stderr[-3000:]
    r = subprocess.run([str(outs["exp3_epilogue_remote"]), "--ndev", "2", "--sizes", "1024x512x256", "--iters", "3", "--warmup", "1", "--verify"],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "FAIL" not in r.stdout and r.stdout.count(" ok") == 3, r.stdout[-3000:] + r.stderr[-3000:]
