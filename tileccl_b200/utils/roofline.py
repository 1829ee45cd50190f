"""Roofline arithmetic for the fused ops.

target time = max(FLOPs / GEMM peak, bytes that must leave each GPU over NVLink / link bandwidth).

Denominators are measurements, read from files, never literals in the code:

* compute: ``MEASURED_PEAKS.json`` at the repository root (a cuBLAS bf16 GEMM timed as a burst and as a
  seconds-long loop under the power cap), else the stated fall-back;
* link: ``peer_copy_gbps`` of the platform file ``utils/platforms/b200_nvswitch.json`` (a large one-direction
  peer copy), or of the file named by ``TILECCL_PLATFORM``.

Which compute peak applies depends on the clock the run held.  A short benchmark on an otherwise idle GPU
runs near the maximum SM clock, where the burst figure is the honest ceiling; a long loop settles at the
power cap, where the sustained one is.  Every result therefore carries both fractions, and
:func:`pick_peak` names the one that matches the sampled clock (burst when the median SM clock under load is
at least 90 % of the maximum).  A fraction above 1 against the sustained peak simply means the run held a
higher clock than the sustained measurement did; it is never reported as the headline.
"""
from __future__ import annotations

import json
import os
from pathlib import Path

FALLBACK = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
_PLATFORM_DEFAULT = Path(__file__).resolve().parent / "platforms" / "b200_nvswitch.json"


def peaks() -> dict:
    p = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    out = dict(FALLBACK)
    out["source"] = "fallback"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            for k in FALLBACK:
                if k in d:
                    out[k] = float(d[k])
            out["source"] = "measured"
        except (OSError, ValueError, TypeError):   # unreadable or malformed file: keep the fallback figures
            out = dict(FALLBACK, source="fallback")
    return out


def link_gbs() -> dict:
    """Measured one-direction peer bandwidth per GPU and where the figure comes from."""
    path = Path(os.environ.get("TILECCL_PLATFORM", str(_PLATFORM_DEFAULT)))
    d = json.loads(path.read_text())
    return {"gbs": float(d["peer_copy_gbps"]), "nominal_gbs": float(d.get("link_nominal_gbps", 0.0)), "file": path.name}


def pick_peak(clocks: dict | None) -> str:
    """'burst' or 'sustained': the compute peak that matches the SM clock a run held under load."""
    if not clocks or not clocks.get("sm_mhz") or not clocks.get("sm_max_mhz"):
        return "sustained"
    return "burst" if float(clocks["sm_mhz"]) >= 0.9 * float(clocks["sm_max_mhz"]) else "sustained"


def _roofline(flops: float, link_bytes: float) -> dict:
    pk, ln = peaks(), link_gbs()
    t_l = link_bytes / (ln["gbs"] * 1e9) * 1e6
    t_b = flops / (pk["bf16_tflops"] * 1e12) * 1e6
    t_s = flops / (pk["bf16_tflops_sustained"] * 1e12) * 1e6
    return {"compute_us": t_s, "compute_burst_us": t_b, "link_us": t_l, "roofline_us": max(t_s, t_l),
            "roofline_burst_us": max(t_b, t_l), "bound": "link" if t_l >= t_s else "compute", "peaks": pk["source"],
            "link_gbs": ln["gbs"], "link_file": ln["file"]}


def gemm_rs_roofline_us(M: int, N: int, K_local: int, world: int) -> dict:
    """Per rank: 2*M*N*K_local FLOPs; (world-1)/world of the [M, N] bf16 partial product leaves the GPU."""
    return _roofline(2.0 * M * N * K_local, (world - 1) / world * M * N * 2 if world > 1 else 0.0)


def ag_gemm_roofline_us(M: int, N_local: int, K: int, world: int) -> dict:
    """Per rank: 2*M*N_local*K FLOPs; (world-1)/world of the gathered [M, K] bf16 activations arrive (and the
    same amount of the rank's own shard leaves)."""
    return _roofline(2.0 * M * N_local * K, (world - 1) / world * M * K * 2 if world > 1 else 0.0)


def fractions(roof: dict, measured_us: float, clocks: dict | None = None) -> dict:
    """Achieved fraction of the roofline against both compute peaks, and the one that applies to this run."""
    if not measured_us or measured_us <= 0:
        return {"pct_burst": None, "pct_sustained": None, "pct": None, "of": None}
    pb = 100.0 * roof["roofline_burst_us"] / measured_us
    ps = 100.0 * roof["roofline_us"] / measured_us
    which = pick_peak(clocks)
    if which == "sustained" and ps > 100.0:
        which = "burst"          # the run held a higher clock than the sustained measurement: only the burst peak bounds it
    return {"pct_burst": round(pb, 1), "pct_sustained": round(ps, 1), "pct": round(pb if which == "burst" else ps, 1), "of": which}


def wave_efficiency(M: int, N: int, cta_group: int = 2, sms: int = 148) -> dict:
    """Share of the persistent grid's tile slots that hold a tile: ``tiles / (waves * groups)``.

    The kernels run one CTA (or CTA pair) per SM over a static list of 128*cta_group x 256 tiles, so
    the last wave is partly empty unless the tile count divides by the number of groups.  This loss is
    part of the distance to the roofline that no kernel tuning removes (the roofline figures above do
    not include it)."""
    tile_m = 128 * cta_group
    tiles = -(-M // tile_m) * -(-N // 256)
    groups = max(1, sms // cta_group)
    waves = -(-tiles // groups)
    return {"tiles": tiles, "groups": groups, "waves": waves, "efficiency": tiles / (waves * groups)}
