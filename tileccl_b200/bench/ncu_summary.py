"""Turns an ncu report into the short text table kept under ``profiles/``.

    ncu -i prof.ncu-rep --page raw --csv > prof.csv        (works without a GPU)
    python -m tileccl_b200.bench.ncu_summary prof.csv [--all]

or directly ``python -m tileccl_b200.bench.ncu_summary prof.ncu-rep`` (runs the ncu import itself).
Prints, per captured launch, the metrics the roofline discussion needs: duration, DRAM bytes and
throughput, tensor-pipe activity, L2 hit rate and throughput, registers, warp occupancy and the top
stall reasons.  The reference reads the same counters by hand from ``ncu --section`` output
(l2_peer_cache/run_all.sh:265-336).
"""
from __future__ import annotations

import csv
import io
import subprocess
import sys

KEEP = [
    "gpu__time_duration.sum", "sm__cycles_elapsed.avg.per_second",
    "sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_elapsed", "sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active",
    "sm__throughput.avg.pct_of_peak_sustained_elapsed", "dram__bytes_read.sum", "dram__bytes_write.sum",
    "gpu__dram_throughput.avg.pct_of_peak_sustained_elapsed", "lts__t_sector_hit_rate.pct", "lts__throughput.avg.pct_of_peak_sustained_elapsed",
    "l1tex__m_xbar2l1tex_read_bytes_mem_global_op_tma_ld.sum", "launch__registers_per_thread", "launch__grid_size", "launch__block_size",
    "sm__warps_active.avg.per_cycle_active",
]
STALL_PREFIX = "smsp__average_warps_issue_stalled_"


def load(path: str) -> list[list[str]]:
    if path.endswith(".ncu-rep"):
        text = subprocess.run(["ncu", "-i", path, "--page", "raw", "--csv"], capture_output=True, text=True, check=True).stdout
    else:
        text = open(path).read()
    return list(csv.reader(io.StringIO(text)))


def summarize(rows: list[list[str]], all_launches: bool = False) -> str:
    if len(rows) < 3:
        return "no launches in the report\n"
    hdr, units, data = rows[0], rows[1], rows[2:]
    col = {h: i for i, h in enumerate(hdr)}
    out = []
    for r in (data if all_launches else data[-1:]):
        name = r[col["Kernel Name"]] if "Kernel Name" in col else "?"
        out.append(f"### {name}")
        out.append("| metric | value |\n|---|---|")
        for k in KEEP:
            if k in col and r[col[k]] != "":
                out.append(f"| {k} | {r[col[k]]} {units[col[k]]} |")
        stalls = []
        for h, i in col.items():
            if h.startswith(STALL_PREFIX) and h.endswith("_per_issue_active.ratio"):
                try:
                    stalls.append((float(r[i]), h[len(STALL_PREFIX):-len("_per_issue_active.ratio")]))
                except ValueError:
                    pass
        stalls.sort(reverse=True)
        if stalls:
            out.append("| top stalls per issue | " + ", ".join(f"{n} {v:.2f}" for v, n in stalls[:4]) + " |")
        out.append("")
    return "\n".join(out) + "\n"


def main(argv=None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    if not argv:
        print(__doc__)
        return 1
    print(summarize(load(argv[0]), "--all" in argv))
    return 0


if __name__ == "__main__":
    sys.exit(main())
