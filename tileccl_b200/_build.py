"""In-tree build of the native code with nvcc for sm_100a.

Everything is compiled into ``tileccl_b200/lib`` (shared library) and
``tileccl_b200/bin`` (stand-alone benchmark programs) so that a snapshot of the
source tree carries the binaries with it; nothing is installed elsewhere and no
JIT cache is used.  The reference builds each program with a per-directory
Makefile (comm_comp/Makefile:12-18, tests/Makefile:12-45); this module plays
that role for the whole tree.

Run ``python -m tileccl_b200._build`` to (re)build; ``build()`` only rebuilds a
target whose sources are newer than its output.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB_DIR = PKG / "lib"
BIN_DIR = PKG / "bin"
OBJ_DIR = PKG / "build"

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--threads", "2"]

# Shared library: sources relative to csrc/.
LIB_NAME = "libtileccl.so"
DEBUG_LIB_NAME = "libtileccl_debug.so"
LIB_SOURCES = [
    "ops/tileccl_ops.cu",
    "runtime/symm_heap.cu",
    "ops/no_alloc.cu",
    "ops/nvls_kernels.cu",
]

# Stand-alone programs: name -> (sources, extra link flags).
PROGRAMS: dict[str, tuple[list[str], list[str]]] = {
    "pk_bw_sweep": (["bench/pk_bw_sweep.cu"], []),
    "sync_cost": (["bench/sync_cost.cu"], []),
    "signal_fanin": (["bench/signal_fanin.cu"], []),
    "peer_l2_probe": (["bench/peer_l2_probe.cu"], []),
    "p2p_ce_vs_tma": (["bench/p2p_ce_vs_tma.cu"], []),
    "pipeline_e2e": (["bench/pipeline_e2e.cu"], []),
    "interference_matrix": (["bench/interference_matrix.cu"], []),
    "intra_sm_matrix": (["bench/intra_sm_matrix.cu"], []),
    "ce_gemm_overlap": (["bench/ce_gemm_overlap.cu"], ["-lcublas"]),
    "exp1_ce_interference": (["bench/exp1_ce_interference.cu"], ["-L", str(LIB_DIR), "-ltileccl", "-Xlinker", "-rpath=$ORIGIN/../lib"]),
    "exp3_gemm_rs_fused": (["bench/exp3_gemm_rs_fused.cu", "runtime/launcher.cpp"], ["-L", str(LIB_DIR), "-ltileccl", "-Xlinker", "-rpath=$ORIGIN/../lib"]),
    "exp2_ag_gemm_granularity": (["bench/exp2_ag_gemm_granularity.cu", "runtime/launcher.cpp"], ["-L", str(LIB_DIR), "-ltileccl", "-Xlinker", "-rpath=$ORIGIN/../lib"]),
    "exp3_epilogue_remote": (["bench/exp3_epilogue_remote.cu", "runtime/launcher.cpp"], ["-L", str(LIB_DIR), "-ltileccl", "-Xlinker", "-rpath=$ORIGIN/../lib"]),
    "host_selftest": (["bench/host_selftest.cpp"], []),
    "launcher_selftest": (["bench/launcher_selftest.cpp", "runtime/launcher.cpp"], []),
}


def nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the native code cannot be built")
    return exe


def _headers() -> list[Path]:
    return [p for p in CSRC.rglob("*") if p.suffix in (".cuh", ".hpp", ".h")]


def _stale(out: Path, srcs: list[Path]) -> bool:
    if not out.exists():
        return True
    t = out.stat().st_mtime
    return any(s.stat().st_mtime > t for s in srcs + _headers())


def _run(cmd: list[str], verbose: bool) -> None:
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"build failed: {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
    if verbose and r.stderr.strip():
        print(r.stderr, flush=True)


def _compile(src: Path, verbose: bool, extra: list[str], tag: str = "") -> Path:
    obj = OBJ_DIR / (str(src.relative_to(CSRC)).replace("/", "_") + tag + ".o")
    if _stale(obj, [src]):
        _run([nvcc(), *ARCH_FLAGS, *COMMON_FLAGS, *extra, "-I", str(CSRC), "-c", str(src), "-o", str(obj)], verbose)
    return obj


def build(verbose: bool = False, programs: bool = True, ptxas_info: bool = False) -> dict[str, Path]:
    """Build the shared library and (optionally) every benchmark program.

    Sources listed above that do not exist yet are skipped, so that the package
    can be built while parts of it are still being written.
    """
    for d in (LIB_DIR, BIN_DIR, OBJ_DIR):
        d.mkdir(exist_ok=True)
    extra = ["-Xptxas", "-v"] if ptxas_info else []
    outputs: dict[str, Path] = {}

    lib_srcs = [CSRC / s for s in LIB_SOURCES if (CSRC / s).exists()]
    lib_out = LIB_DIR / LIB_NAME
    with ThreadPoolExecutor(max_workers=max(1, min(8, os.cpu_count() or 1))) as ex:
        objs = list(ex.map(lambda s: _compile(s, verbose, extra), lib_srcs))
        if _stale(lib_out, objs) or any(o.stat().st_mtime > lib_out.stat().st_mtime for o in objs):
            _run([nvcc(), *ARCH_FLAGS, "-shared", "-o", str(lib_out), *map(str, objs)], verbose)
        outputs[LIB_NAME] = lib_out
        # Debug variant: the same sources with device-side address checks (TCL_DEBUG_BOUNDS).
        dbg_out = LIB_DIR / DEBUG_LIB_NAME
        dobjs = list(ex.map(lambda s: _compile(s, verbose, extra + ["-DTCL_DEBUG_BOUNDS"], ".dbg"), lib_srcs))
        if _stale(dbg_out, dobjs) or any(o.stat().st_mtime > dbg_out.stat().st_mtime for o in dobjs):
            _run([nvcc(), *ARCH_FLAGS, "-shared", "-o", str(dbg_out), *map(str, dobjs)], verbose)
        outputs[DEBUG_LIB_NAME] = dbg_out

        if programs:
            def one(item):
                name, (srcs, link) = item
                paths = [CSRC / s for s in srcs]
                if not all(p.exists() for p in paths):
                    return None
                out = BIN_DIR / name
                if _stale(out, paths):
                    os_ = [_compile(p, verbose, extra) for p in paths]
                    _run([nvcc(), *ARCH_FLAGS, "-o", str(out), *map(str, os_), *link], verbose)
                return name, out

            for res in ex.map(one, PROGRAMS.items()):
                if res:
                    outputs[res[0]] = res[1]
    return outputs


if __name__ == "__main__":
    outs = build(verbose=True, ptxas_info="--ptxas" in sys.argv)
    for k, v in outs.items():
        print(f"{k}: {v}")
