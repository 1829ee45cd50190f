"""Transport selector: the decision table of the probe suite as code.

The reference ends its analysis with a decision table (which transport for which situation) and a
vector of platform parameters that an automatic chooser would need, and lists "encode the table
as a back-end selector plus one parameter file per platform" as its next milestone
(tests/ANALYSIS.md:118-173).  This module is that selector for B200 / NVLink 5 / NVSwitch.

The parameters are the figures this suite measured on 8 x B200 (``reports/REPORT_b200.md`` gives the
runs): ``pk_bw_sweep`` (link bandwidth per mover, SMs to saturate, per-copy cost of the copy engine),
``p2p_ce_vs_tma`` (one-shot latencies), ``sync_cost`` (one-way latency, cost of a release flag),
``interference_matrix`` / ``exp1_ce_interference`` (what a transfer costs a concurrent kernel).
Another platform overrides them with ``Platform.from_json``; ``utils/platforms/`` holds this B200 vector and,
for comparison, the two machines of the reference filled in from the figures it publishes.

Limits: the link figures are those of one transfer between one pair of GPUs.  When every GPU sends to
every other at once the copy engines reach less (462 GB/s per GPU in exp1's 56-leg all-gather pattern),
and the model knows nothing of data dependencies: a transfer that must wait for a kernel's tiles is not
"independent".  It ranks transports for a planner; it does not replace measuring the fused kernel.

The model is the zero-parameter one the reference validates with ``pipeline_e2e``:
a pipelined producer -> transfer -> consumer takes ``max(Tc_src, Tm, Tc_dst)``; a transfer takes
``start + n_msgs * per_message + bytes / bandwidth``; a transport that occupies SMs slows an SM-bound
kernel by the share of SMs it takes, one that does not by its measured interference factor.
"""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass, field

TRANSPORTS = ("ce", "reg", "bulk", "fused_st", "fused_pull")


@dataclass
class Platform:
    name: str = "B200 NVLink5 NVSwitch"
    notes: str = ""                   # where the figures come from, which ones are placeholders
    sms: int = 148
    # link bandwidth per direction, GB/s
    ce_gbps: float = 749.0            # copy engine, 128 MB copy
    peer_copy_gbps: float = 770.0     # large one-direction peer copy: the link denominator of the rooflines (utils/roofline.py)
    peer_copy_source: str = ""        # where that figure was measured
    link_nominal_gbps: float = 900.0  # the link's nominal rate per direction, for context
    sm_gbps: float = 700.0            # register or bulk-copy mover, any message >= 2 KB
    per_sm_gbps: float = 50.0         # what one SM of a mover sustains; 16 SMs saturate the link
    fused_st_gbps: float = 620.0      # 16-byte peer stores from a GEMM epilogue (all-to-all pattern)
    fused_pull_gbps: float = 705.0    # peer loads by gather warps of all SMs
    # fixed costs, microseconds
    ce_per_copy_us: float = 3.7       # each cudaMemcpyPeerAsync beyond its bytes
    launch_us: float = 4.0            # a mover kernel of its own
    one_way_us: float = 2.6           # store becomes visible at the peer
    flag_us: float = 1.45             # release flag after a payload (st.release, fence + st, red.release alike)
    min_msg_reg: int = 512            # below this a message no longer reaches sm_gbps
    min_msg_bulk: int = 2048
    # slow-down of a concurrent kernel (S_c) when the transfer does not take its SMs, by what bounds the kernel
    # (interference_matrix, probe on 132 SMs and mover on 16; "tensor" for ce is exp1's GEMM under 7 pull legs)
    s_c: dict = field(default_factory=lambda: {
        "ce": {"tensor": 1.03, "hbm": 1.01, "l2": 1.14},
        "reg": {"tensor": 1.01, "hbm": 1.06, "l2": 1.25},
        "bulk": {"tensor": 1.00, "hbm": 1.03, "l2": 1.97},
        "fused_st": {"tensor": 1.00, "hbm": 1.06, "l2": 1.25},
        "fused_pull": {"tensor": 1.00, "hbm": 1.06, "l2": 1.25},
    })
    # slow-down of the transfer itself (S_m) under that kernel
    s_m: dict = field(default_factory=lambda: {
        "ce": {"tensor": 1.00, "hbm": 1.08, "l2": 1.01},
        "reg": {"tensor": 1.02, "hbm": 1.09, "l2": 1.01},
        "bulk": {"tensor": 1.02, "hbm": 1.19, "l2": 1.02},
        "fused_st": {"tensor": 1.00, "hbm": 1.09, "l2": 1.01},
        "fused_pull": {"tensor": 1.00, "hbm": 1.09, "l2": 1.01},
    })

    @classmethod
    def from_json(cls, path: str) -> "Platform":
        with open(path) as f:
            d = json.load(f)
        base = asdict(cls())
        unknown = set(d) - set(base)
        if unknown:
            raise ValueError(f"unknown platform parameters: {sorted(unknown)}")
        base.update(d)
        return cls(**base)

    def to_json(self, path: str) -> None:
        with open(path, "w") as f:
            json.dump(asdict(self), f, indent=1)


def load_platform(name: str) -> Platform:
    """A parameter file shipped with the package (``b200_nvswitch``, ``h20_nvlink_reference``, ``rtx_pcie5_reference``)."""
    import os
    return Platform.from_json(os.path.join(os.path.dirname(os.path.abspath(__file__)), "platforms", name + ".json"))


def transfer_us(p: Platform, transport: str, nbytes: int, n_msgs: int = 1, sms: int = 16) -> float:
    """Time of one transfer of ``nbytes`` split in ``n_msgs`` equal messages."""
    if transport not in TRANSPORTS:
        raise ValueError(f"unknown transport {transport!r}")
    if nbytes <= 0:
        return 0.0
    n_msgs = max(1, n_msgs)
    msg = nbytes / n_msgs
    if transport == "ce":
        return n_msgs * p.ce_per_copy_us + nbytes / (p.ce_gbps * 1e3) + p.one_way_us
    if transport in ("reg", "bulk"):
        bw = min(p.sm_gbps, p.per_sm_gbps * max(1, sms))
        floor = p.min_msg_reg if transport == "reg" else p.min_msg_bulk
        if msg < floor:                      # short messages: the per-message issue cost shows
            bw *= msg / floor
        return p.launch_us + nbytes / (bw * 1e3) + p.one_way_us
    bw = p.fused_st_gbps if transport == "fused_st" else p.fused_pull_gbps
    return nbytes / (bw * 1e3) + p.one_way_us + p.flag_us      # no launch: it rides in the compute kernel


def compute_slowdown(p: Platform, transport: str, bound: str = "tensor", sms: int = 16) -> float:
    """Factor by which a kernel bound by ``bound`` (tensor, hbm, l2) slows while the transfer runs."""
    if bound not in ("tensor", "hbm", "l2"):
        raise ValueError("bound must be tensor, hbm or l2")
    f = p.s_c[transport][bound]
    if transport in ("reg", "bulk") and bound == "tensor":
        f *= p.sms / max(1, p.sms - sms)     # a mover kernel of its own takes whole SMs from an SM-bound kernel
    return f


def pipeline_us(tc_src: float, tm: float, tc_dst: float) -> float:
    """Steady-state time of a tile pipeline producer -> transfer -> consumer."""
    return max(tc_src, tm, tc_dst)


def choose(p: Platform, nbytes: int, n_msgs: int = 1, compute_us: float = 0.0, bound: str = "tensor",
           fused_possible: bool = False, sms_spare: int = 16) -> dict:
    """Ranks the transports for moving ``nbytes`` while a kernel of ``compute_us`` runs.

    Returns ``{"best": name, "table": {name: {"comm_us", "compute_us", "total_us"}}}`` where total is the
    overlapped time ``max(comm, slowed compute)``.  ``fused_possible`` says the data is produced or consumed
    by a kernel that can carry the transfer itself (epilogue stores, gather warps).
    """
    table = {}
    for t in TRANSPORTS:
        if t.startswith("fused") and not fused_possible:
            continue
        if t in ("reg", "bulk") and sms_spare <= 0:
            continue
        comm = transfer_us(p, t, nbytes, n_msgs, sms_spare) * (p.s_m[t][bound] if compute_us > 0 else 1.0)
        comp = compute_us * compute_slowdown(p, t, bound, sms_spare) if compute_us > 0 else 0.0
        table[t] = {"comm_us": comm, "compute_us": comp, "total_us": max(comm, comp)}
    best = min(table, key=lambda k: (table[k]["total_us"], table[k]["comm_us"]))
    return {"best": best, "table": table}


def main(argv=None) -> int:
    """``python -m tileccl_b200.utils.selector --bytes 64M [--msgs N] [--compute-us T --bound tensor|hbm|l2]
    [--fused] [--sms 16] [--platform NAME|FILE.json]`` prints the ranking."""
    import argparse
    ap = argparse.ArgumentParser(description=main.__doc__)
    ap.add_argument("--bytes", required=True)
    ap.add_argument("--msgs", type=int, default=1)
    ap.add_argument("--compute-us", type=float, default=0.0)
    ap.add_argument("--bound", default="tensor", choices=["tensor", "hbm", "l2"])
    ap.add_argument("--fused", action="store_true", help="the producing or consuming kernel can carry the transfer")
    ap.add_argument("--sms", type=int, default=16, help="SMs a mover kernel may take")
    ap.add_argument("--platform", default="b200_nvswitch")
    a = ap.parse_args(argv)
    mult = {"K": 1 << 10, "M": 1 << 20, "G": 1 << 30}
    txt = a.bytes.strip().upper().rstrip("B")
    nbytes = int(float(txt[:-1]) * mult[txt[-1]]) if txt and txt[-1] in mult else int(txt)
    p = Platform.from_json(a.platform) if a.platform.endswith(".json") else load_platform(a.platform)
    r = choose(p, nbytes, a.msgs, a.compute_us, a.bound, a.fused, a.sms)
    print(f"# {p.name}: {nbytes} bytes in {a.msgs} message(s)" + (f", beside a {a.bound}-bound kernel of {a.compute_us:.0f} us" if a.compute_us else ""))
    print(f"{'transport':12s} {'comm us':>10s} {'compute us':>11s} {'total us':>10s}")
    for t, v in sorted(r["table"].items(), key=lambda kv: kv[1]["total_us"]):
        print(f"{t:12s} {v['comm_us']:10.1f} {v['compute_us']:11.1f} {v['total_us']:10.1f}" + ("   <- best" if t == r["best"] else ""))
    return 0


if __name__ == "__main__":
    import sys
    sys.exit(main())
