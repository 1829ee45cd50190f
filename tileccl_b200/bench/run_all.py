"""Suite orchestrator: environment snapshot, pre-flight check, build, GPU sampler, under-load clock
check, every experiment with its own time-out, manifest, verdicts, zip bundle.

    python -m tileccl_b200.bench.run_all --out reports/results_$(date +%Y%m%d_%H%M%S) [--quick] [--resume DIR]

Reads but never changes GPU settings: clocks are sampled and reported, not locked (the reference's
run_all.sh aborts unless clocks are held with ``nvidia-smi -lgc``; here every experiment takes its
baselines paired and interleaved instead, and the bundle records the clocks seen under load).

Bundle layout (same as the reference's): manifest.txt (one line per step: name, rc, seconds),
env.txt, build.log, <step>.log, *.csv, gpu_trace.csv, clocks_after.txt, verdict.txt, and a zip.
``--resume DIR`` re-runs only the steps whose manifest line is missing or has rc != 0.

Reference parity: comm_comp/run_all.sh (env :36-52, pre-check :60-90, sampler :110-141, run :146-159,
QUICK presets :176-191, load clock check :208-258, experiment list :267-333), l2_peer_cache/run_all.sh
(probe sweeps :202-256, verdict :386-516), comm_comp/rerun_m32768.sh (M / K / order sweeps :148-212).
"""
from __future__ import annotations

import argparse
import os
import shutil
import signal
import subprocess
import sys
import time
import zipfile
from pathlib import Path

PKG = Path(__file__).resolve().parents[1]
BIN = PKG / "bin"


def sh(cmd: str, timeout: float = 60.0) -> str:
    try:
        r = subprocess.run(cmd, shell=True, capture_output=True, text=True, timeout=timeout)
        return (r.stdout + r.stderr).strip()
    except Exception as e:  # noqa: BLE001
        return f"<{cmd}: {e}>"


def env_snapshot(out: Path) -> None:
    parts = [
        ("date", "date -u"), ("uname", "uname -a"), ("git", f"git -C {PKG.parent} log -1 --format='%H %s' 2>/dev/null"),
        ("nvcc", "nvcc --version | tail -2"), ("python", f"{sys.executable} -c 'import torch,sys;print(sys.version.split()[0], torch.__version__)'"),
        ("nvidia-smi", "nvidia-smi"), ("topology", "nvidia-smi topo -m"),
        ("clocks", "nvidia-smi --query-gpu=index,name,clocks.sm,clocks.max.sm,clocks.mem,power.limit,persistence_mode --format=csv"),
        ("nvlink", "nvidia-smi nvlink -s | head -40"), ("cpu", "lscpu | head -20"),
    ]
    with open(out / "env.txt", "w") as f:
        for name, cmd in parts:
            f.write(f"==== {name}: {cmd}\n{sh(cmd)}\n\n")


def gpu_count() -> int:
    try:
        import torch
        return torch.cuda.device_count() if torch.cuda.is_available() else 0
    except Exception:  # noqa: BLE001
        return 0


def precheck(log, force: bool) -> bool:
    """GPUs should be idle; clocks are reported as found (read-only)."""
    q = sh("nvidia-smi --query-gpu=index,utilization.gpu,memory.used,clocks.sm,clocks.max.sm --format=csv,noheader,nounits")
    ok = True
    for line in q.splitlines():
        p = [x.strip() for x in line.split(",")]
        if len(p) < 5:
            continue
        try:
            util, mem = float(p[1]), float(p[2])
        except ValueError:
            continue
        if util > 10 or mem > 4096:
            log(f"pre-check: GPU {p[0]} is busy (util {util} %, {mem} MiB used)")
            ok = False
    if not ok and not force:
        log("pre-check failed: another job is using the GPUs (use --force to run anyway)")
    return ok or force


class Sampler:
    """100 ms nvidia-smi trace of every GPU for the whole run."""

    def __init__(self, path: Path):
        self.proc = None
        exe = shutil.which("nvidia-smi")
        if exe:
            self.proc = subprocess.Popen(
                [exe, "--query-gpu=timestamp,index,clocks.sm,clocks.mem,power.draw,temperature.gpu,utilization.gpu,"
                      "clocks_event_reasons.active", "--format=csv", "-lms", "100"],
                stdout=open(path, "w"), stderr=subprocess.DEVNULL)

    def stop(self):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:  # noqa: BLE001
                self.proc.kill()


_running: dict = {"proc": None}      # the step in flight, for the signal handler


def end_group(p, grace: float = 30.0) -> None:
    """Ends a step's whole process group (the launcher and every rank): SIGINT first, SIGKILL after ``grace``."""
    try:
        os.killpg(p.pid, signal.SIGINT)
    except ProcessLookupError:
        return
    try:
        p.wait(timeout=grace)
    except subprocess.TimeoutExpired:
        os.killpg(p.pid, signal.SIGKILL)
        p.wait()


def install_signal_handlers(log) -> None:
    """A step runs in a session of its own, so a signal that ends the orchestrator would leave its ranks behind,
    still holding the GPUs.  SIGTERM / SIGINT / SIGHUP therefore end the running step's process group first."""
    def handler(signum, _frame):
        p = _running["proc"]
        log(f"signal {signum}: ending the running step and leaving")
        if p is not None and p.poll() is None:
            end_group(p, grace=10.0)
        raise SystemExit(128 + signum)
    for sig in (signal.SIGTERM, signal.SIGINT, signal.SIGHUP):
        signal.signal(sig, handler)


def run_step(name: str, cmd: list[str], timeout: float, out: Path, log, manifest: bool = True) -> int:
    """Runs one experiment in its own process group; on time-out the group (and only it) is killed.
    ``manifest=False``: the command writes the manifest lines of its parts itself (a batched launch)."""
    t0 = time.time()
    with open(out / f"{name}.log", "w") as lf:
        lf.write("$ " + " ".join(cmd) + "\n")
        lf.flush()
        p = subprocess.Popen(cmd, stdout=lf, stderr=subprocess.STDOUT, cwd=str(PKG.parent), start_new_session=True)
        _running["proc"] = p
        try:
            rc = p.wait(timeout=timeout)
        except subprocess.TimeoutExpired:
            end_group(p)
            rc = 124
        finally:
            _running["proc"] = None
    dur = time.time() - t0
    if manifest or rc != 0:
        with open(out / "manifest.txt", "a") as mf:
            mf.write(f"{name} rc={rc} seconds={dur:.1f}\n")
    log(f"  {name}: rc={rc} in {dur:.1f} s")
    return rc


def done_steps(out: Path) -> set[str]:
    ok = set()
    mf = out / "manifest.txt"
    if mf.exists():
        for line in mf.read_text().splitlines():
            parts = line.split()
            if len(parts) >= 2 and parts[1] == "rc=0":
                ok.add(parts[0])
            elif parts:
                ok.discard(parts[0])
    return ok


class RankCmd(list):
    """Command line of a step that runs one process per GPU through ``tileccl_b200.launch``; ``tail`` is the
    experiment module and its flags, which is what a batched run strings together with ``--then``."""

    def __init__(self, prefix: list[str], tail: list[str]):
        super().__init__(prefix + tail)
        self.tail = list(tail)

    def __add__(self, other):
        return RankCmd(list(self)[: len(self) - len(self.tail)], self.tail + list(other))


def plan(n_gpus: int, quick: bool, out: Path, tuning: bool = False, iters: int = 0) -> list[tuple[str, list[str], float, int]]:
    """(step name, command, time-out seconds, GPUs needed).  ``iters`` > 0 overrides the iteration count of
    the fused experiments (100 in a full run, 10 in a quick one)."""
    py = sys.executable
    launch = RankCmd([py, "-m", "tileccl_b200.launch", "-n", str(max(1, n_gpus))], [])
    o = str(out)
    it = str(iters) if iters > 0 else ("10" if quick else "100")
    it2 = str(iters) if iters > 0 else ("10" if quick else "30")      # the longer-running experiments take fewer iterations
    steps = []
    # ---- fused ops (Python drivers, one process per GPU) ----
    m_sweep = ["8192", "32768"] if quick else ["512", "1024", "2048", "4096", "8192", "16384", "32768"]
    for m in m_sweep:
        steps.append((f"exp3_fused_m{m}", launch + ["exp3_gemm_rs_fused", "--m", m, "--n", "8192", "--k-global", "8192", "--iters", it, "--verify",
                                                    "--csv", f"{o}/exp3_fused_msweep.csv", "--dump-iters", f"{o}/iters_m{m}"], 600, 2))
    for k in (["1024"] if quick else ["512", "2048", "8192"]):
        steps.append((f"exp3_fused_k{k}", launch + ["exp3_gemm_rs_fused", "--m", "8192", "--n", "8192", "--k", k, "--iters", it, "--csv", f"{o}/exp3_fused_ksweep.csv"], 600, 2))
    if not quick:
        for order in ("fused,ctrl,base,nccl", "ctrl,base,fused,nccl"):
            steps.append((f"exp3_order_{order.split(',')[0]}", launch + ["exp3_gemm_rs_fused", "--m", "32768", "--n", "8192", "--k-global", "8192", "--iters", it,
                                                                        "--order", order, "--csv", f"{o}/exp3_order.csv"], 600, 2))
    steps.append(("exp3_epilogue", launch + ["exp3_epilogue_remote", "--sizes", "8192,32768x8192x1024" if quick else "8192,8192x8192x512,512x8192x8192,32768x8192x8192,32768x8192x1024",
                                             "--iters", it, "--verify", "--csv", f"{o}/exp3_epilogue.csv"] + ([] if quick else ["--epi", "st16,st256,tma"]), 900, 2))
    steps.append(("exp2_ag_gemm", launch + ["exp2_ag_gemm_granularity", "--m", "32768", "--k", "8192", "--n-global", "28672", "--gather-rows", "512,4096" if quick else "128,512,2048,4096",
                                            "--iters", it2, "--verify", "--csv", f"{o}/exp2.csv"], 1200, 2))
    steps.append(("nvls_bw", launch + ["nvls_bw", "--csv", f"{o}/nvls_bw.csv"] + (["--sizes", "64K,16M,256M", "--iters", "10"] if quick else []), 600, 2))
    steps.append(("exp3_fused_nvls", launch + ["exp3_gemm_rs_fused", "--m", "32768", "--n", "8192", "--k-global", "8192", "--iters", it, "--transport", "nvls", "--verify",
                                                "--csv", f"{o}/exp3_fused_nvls.csv"], 600, 2))
    steps.append(("mlp_e2e", launch + ["mlp_e2e", "--iters", it2 if iters > 0 or quick else "50", "--verify", "--csv", f"{o}/mlp_e2e.csv"], 900, 1))
    if tuning:
        # knob sweeps of both fused ops at the headline shapes: all settings in one process per rank, timed in turn.
        # Dozens of plans live side by side in it, so it runs as a launch of its own (a plain list is never batched).
        steps.append(("tune_fused", list(launch + ["tune_fused", "--ops", "rs,ag", "--m", "32768", "--n", "8192", "--k-global", "8192", "--iters", it2,
                                                   "--csv", f"{o}/exp3_tuning.csv"]), 150, 2))
    steps.append(("bench", [py, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={max(1, n_gpus)}", "--master-addr", "127.0.0.1", "--master-port", "29571",
                            "bench.py", "--gpus", str(max(1, n_gpus)), "--steps", it2, "--warmup", "5"], 900, 1))
    # ---- C++ programs (single process, several GPUs) ----
    b = lambda n: str(BIN / n)  # noqa: E731
    steps.append(("exp3_fused_native", [b("exp3_gemm_rs_fused"), "--m", "32768", "--n", "8192", "--k-global", "8192", "--iters", it, "--verify", "--csv", f"{o}/exp3_fused_native.csv"], 600, 2))
    steps.append(("exp2_native", [b("exp2_ag_gemm_granularity"), "--gather-rows", "512,4096" if quick else "128,512,2048,4096", "--iters", "8" if quick else "30", "--verify", "--csv", f"{o}/exp2_native.csv"], 900, 2))
    steps.append(("exp3_epilogue_native", [b("exp3_epilogue_remote"), "--iters", it, "--verify", "--csv", f"{o}/exp3_epilogue_native.csv"], 600, 2))
    steps.append(("exp1_ce_interference", [b("exp1_ce_interference"), "--sizes", "8192" if quick else "2048,4096,8192", "--iters", "10" if quick else "30", "--csv", f"{o}/exp1.csv"], 900, 2))
    steps.append(("pk_bw_sweep", [b("pk_bw_sweep"), "--total", "256M" if quick else "1G", "--csv", f"{o}/pk_bw.csv"], 900, 2))
    steps.append(("p2p_ce_vs_tma", [b("p2p_ce_vs_tma"), "--csv", f"{o}/p2p_ce_vs_tma.csv"] + (["--tokens", "1,64,4096", "--iters", "20"] if quick else []), 600, 2))
    steps.append(("sync_cost", [b("sync_cost"), "--csv", f"{o}/sync_cost.csv"], 300, 2))
    steps.append(("signal_fanin", [b("signal_fanin"), "--csv", f"{o}/signal_fanin.csv"] + (["--fanin", "1,4,32", "--rounds", "50"] if quick else ["--fanin", "1,2,3,4,5,6,7,16,32", "--sizes", "4K,32K,128K,1M,4M"]), 900, 2))
    steps.append(("pipeline_e2e", [b("pipeline_e2e"), "--csv", f"{o}/pipeline_e2e.csv"] + (["--intensity", "0,256", "--reps", "2"] if quick else []), 900, 2))
    steps.append(("interference_matrix", [b("interference_matrix"), "--csv", f"{o}/interference.csv"] + (["--window-ms", "100", "--iters", "5"] if quick else []), 900, 2))
    steps.append(("interference_dst", [b("interference_matrix"), "--probe-dev", "dst", "--csv", f"{o}/interference.csv"] + (["--window-ms", "100", "--iters", "5"] if quick else []), 900, 2))
    steps.append(("interference_starve", [b("interference_matrix"), "--mode", "starve", "--total", "64M", "--csv", f"{o}/interference.csv"], 300, 2))
    steps.append(("intra_sm_matrix", [b("intra_sm_matrix"), "--csv", f"{o}/intra_sm.csv"] + (["--window-ms", "100", "--comm-warps", "1,4"] if quick else []), 900, 2))
    steps.append(("intra_sm_concentrated", [b("intra_sm_matrix"), "--comm-ctas", "8", "--csv", f"{o}/intra_sm.csv"] + (["--window-ms", "100", "--comm-warps", "4"] if quick else []), 900, 2))
    steps.append(("ce_gemm_overlap", [b("ce_gemm_overlap"), "--csv", f"{o}/ce_gemm_overlap.csv"] + (["--sizes", "8192", "--iters", "10"] if quick else []), 900, 1))
    # ---- peer-L2 probe: both L1 policies x (via, dir) cells + a big-buffer calibration point ----
    tot = ["--total", "1G", "--reps", "3"] if quick else []
    for cache in ("ca", "cg"):
        steps.append((f"l2_probe_{cache}", [b("peer_l2_probe"), "--cache", cache, "--csv", f"{o}/probe_{cache}"] + tot, 900, 2))
    steps.append(("l2_probe_st", [b("peer_l2_probe"), "--modes", "bw", "--dir", "write", "--csv", f"{o}/probe_st"] + tot, 600, 2))
    steps.append(("l2_probe_tma", [b("peer_l2_probe"), "--modes", "bw", "--via", "tma", "--csv", f"{o}/probe_tma"] + tot, 600, 2))
    steps.append(("l2_probe_tmast", [b("peer_l2_probe"), "--modes", "bw", "--via", "tma", "--dir", "write", "--csv", f"{o}/probe_tmast"] + tot, 600, 2))
    steps.append(("l2_wire_bigbuf", [b("peer_l2_probe"), "--modes", "wire", "--wire-sizes", "512M", "--csv", f"{o}/probe_bigbuf"] + (["--wire-total", "4G"] if quick else []), 600, 2))
    steps.append(("launcher_selftest", [b("launcher_selftest"), "--mode", "ok", "--world", "4"], 60, 0))
    return steps


def batch_rank_steps(steps, out: Path):
    """Merges runs of consecutive one-process-per-GPU steps into one launch each: the experiments then share one
    set of rank processes (one interpreter start and one rendezvous instead of one per step).  ``bench/run.py``
    writes each experiment's own manifest line and log, so the bundle looks the same as an unbatched one."""
    merged, run = [], []

    def flush():
        if not run:
            return
        if len(run) == 1:
            merged.append(run[0])
        else:
            head = run[0][1]
            prefix = list(head)[: len(head) - len(head.tail)]
            tail = ["--manifest", str(out / "manifest.txt"), "--logs", str(out)]
            for i, (name, cmd, _to, _need) in enumerate(run):
                tail += (["--then"] if i else []) + cmd.tail + ["--as", name]
            # the parts' own limits are generous; a whole batch gets at most a quarter of their sum (and at least ten minutes)
            limit = max(600.0, 0.25 * sum(t for _, _, t, _ in run))
            merged.append((f"batch_{run[0][0]}..{run[-1][0]}", prefix + tail, limit, max(n for _, _, _, n in run)))
        run.clear()

    for st in steps:
        if isinstance(st[1], RankCmd):
            run.append(st)
        else:
            flush()
            merged.append(st)
    flush()
    return merged


def scrub_paths(out: Path) -> None:
    """Rewrites the text files of a bundle so that they name no directory of the machine that made them: the
    bundle's own path becomes ``<bundle>``, the source tree ``<repo>`` and the interpreter ``python``."""
    subs = [(str(out), "<bundle>"), (str(PKG.parent.resolve()), "<repo>"), (str(PKG.parent), "<repo>"), (sys.executable, "python"),
            (os.path.realpath(sys.executable), "python")]
    subs = sorted(set(s for s in subs if s[0]), key=lambda kv: -len(kv[0]))
    for p in out.rglob("*"):
        if not p.is_file() or p.suffix not in (".log", ".txt", ".csv", ".md"):
            continue
        try:
            text = p.read_text()
        except (UnicodeDecodeError, OSError):
            continue
        new = text
        for a, b in subs:
            new = new.replace(a, b)
        if new != text:
            p.write_text(new)


def load_clock_check(out: Path, log) -> None:
    """Records what the SM clock does under a sustained GEMM (read-only: nothing is locked)."""
    code = ("import torch,time;a=torch.randn(8192,8192,device='cuda',dtype=torch.bfloat16);b=a.clone();"
            "t=time.time()\nwhile time.time()-t<4: torch.matmul(a,b)\ntorch.cuda.synchronize()")
    from ..utils.clocks import ClockSampler
    s = ClockSampler(period_ms=100, gpu_index=0).start()
    subprocess.run([sys.executable, "-c", code], capture_output=True, timeout=120)
    summ = s.summary()
    (out / "load_clock_check.txt").write_text(str(summ) + "\n")
    log(f"under-load clocks on GPU 0: {summ}")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--out", default=None)
    ap.add_argument("--resume", default=None, help="existing bundle: re-run only steps that did not finish with rc=0")
    ap.add_argument("--quick", action="store_true")
    ap.add_argument("--force", action="store_true", help="run even if the pre-check finds the GPUs busy")
    ap.add_argument("--only", default=None, help="comma list of step-name prefixes")
    ap.add_argument("--list", action="store_true")
    ap.add_argument("--tuning", action="store_true", help="add the knob sweeps of the two fused ops (step tune_fused, CSV exp3_tuning.csv)")
    ap.add_argument("--iters", type=int, default=0, help="iteration count of the fused experiments (default: 100, or 10 with --quick)")
    ap.add_argument("--batch", action="store_true", help="run consecutive one-process-per-GPU experiments in one set of rank processes")
    ap.add_argument("--keep", action="store_true", help="do not zip the bundle")
    ap.add_argument("--ncu", action="store_true", help="also capture the NVLink section of one peer_l2_probe launch with ncu (off by default; needs profiling permission)")
    args = ap.parse_args(argv)
    out = Path(args.resume or args.out or f"reports/results_{time.strftime('%Y%m%d_%H%M%S')}").resolve()
    n = gpu_count()
    steps = plan(n, args.quick, out, tuning=args.tuning, iters=args.iters)
    if args.ncu and shutil.which("ncu"):
        # One small single-launch capture, one GPU's kernel, clocks left alone.  The plain command runs first.
        once = [str(BIN / "peer_l2_probe"), "--modes", "once", "--targets", "peer", "--sizes", "256M", "--total", "1G", "--no-verify"]
        steps.append(("l2_once_plain", once, 120, 2))
        steps.append(("l2_once_ncu", ["ncu", "--section", "Nvlink", "--section", "MemoryWorkloadAnalysis", "--clock-control", "none", "-k", "regex:stream_read",
                                      "-c", "1", "-o", f"{out}/l2_once", "-f"] + once, 300, 2))
    if args.only:
        pre = [p.strip() for p in args.only.split(",")]
        steps = [s for s in steps if any(s[0].startswith(p) for p in pre)]
    if args.list:
        for name, cmd, to, need in steps:
            print(f"{name:28s} gpus>={need} timeout={to:.0f}s  {' '.join(cmd)}")
        return 0
    out.mkdir(parents=True, exist_ok=True)

    def log(msg: str) -> None:
        line = f"[{time.strftime('%H:%M:%S')}] {msg}"
        print(line, flush=True)
        with open(out / "run.log", "a") as f:
            f.write(line + "\n")

    log(f"bundle {out}  gpus={n} quick={args.quick} resume={bool(args.resume)}")
    install_signal_handlers(log)
    env_snapshot(out)
    if n and not precheck(log, args.force):
        return 2
    from .. import _build
    try:
        outs = _build.build(verbose=False)
        (out / "build.log").write_text("\n".join(f"{k}: {v}" for k, v in outs.items()) + "\n")
    except Exception as e:  # noqa: BLE001
        (out / "build.log").write_text(str(e))
        log("build failed")
        return 3
    sampler = Sampler(out / "gpu_trace.csv") if n else None
    try:
        if n and not args.resume:
            load_clock_check(out, log)
        skip = done_steps(out) if args.resume else set()
        worst = 0
        todo = []
        for name, cmd, to, need in steps:
            if name in skip:
                log(f"  {name}: already done, skipped")
                continue
            if n < need:
                with open(out / "manifest.txt", "a") as mf:
                    mf.write(f"{name} rc=skipped needs={need}gpus\n")
                log(f"  {name}: skipped (needs {need} GPUs, have {n})")
                continue
            todo.append((name, cmd, to, need))
        if args.batch:
            todo = batch_rank_steps(todo, out)
        for name, cmd, to, need in todo:
            worst = max(worst, run_step(name, cmd, to, out, log, manifest=not name.startswith("batch_")))
    finally:
        if sampler:
            sampler.stop()
    (out / "clocks_after.txt").write_text(sh("nvidia-smi --query-gpu=index,clocks.sm,clocks.max.sm,clocks_event_reasons.active --format=csv") + "\n")
    from . import analyze
    try:
        (out / "verdict.txt").write_text(analyze.report(str(out)))
    except Exception as e:  # noqa: BLE001
        (out / "verdict.txt").write_text(f"analysis failed: {e}\n")
    log(f"done, worst rc {worst}")
    scrub_paths(out)
    if not args.keep:
        with zipfile.ZipFile(str(out) + ".zip", "w", zipfile.ZIP_DEFLATED) as z:
            for p in sorted(out.rglob("*")):
                if p.is_file():
                    z.write(p, p.relative_to(out.parent))
    return 0 if worst == 0 else 1


if __name__ == "__main__":
    sys.exit(main())
