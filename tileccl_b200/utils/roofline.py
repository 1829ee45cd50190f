"""Roofline arithmetic for the fused ops.

Denominators come from ``MEASURED_PEAKS.json`` at the repository root when it
exists (a measured STREAM-style copy and cuBLAS bf16 GEMM on this pool's
B200s); otherwise from the stated fall-back.  NVLink uses the measured peer
copy bandwidth per direction.  target time = max(FLOPs / GEMM peak, bytes that
must cross NVLink per GPU / link bandwidth).
"""
from __future__ import annotations

import json
from pathlib import Path

FALLBACK = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
NVLINK_GBS_PER_DIR = 770.0       # measured peer copy, per direction per GPU
NVLINK_GBS_NOMINAL = 900.0


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


def gemm_rs_roofline_us(M: int, N: int, K_local: int, world: int, sustained: bool = True) -> dict:
    pk = peaks()
    tf = pk["bf16_tflops_sustained" if sustained else "bf16_tflops"]
    flops = 2.0 * M * N * K_local
    link_bytes = (world - 1) / world * M * N * 2 if world > 1 else 0.0
    t_c = flops / (tf * 1e12) * 1e6
    t_l = link_bytes / (NVLINK_GBS_PER_DIR * 1e9) * 1e6
    return {"compute_us": t_c, "link_us": t_l, "roofline_us": max(t_c, t_l), "peaks": pk["source"]}


def ag_gemm_roofline_us(M: int, N_local: int, K: int, world: int, sustained: bool = True) -> dict:
    pk = peaks()
    tf = pk["bf16_tflops_sustained" if sustained else "bf16_tflops"]
    flops = 2.0 * M * N_local * K
    link_bytes = (world - 1) / world * M * K * 2 if world > 1 else 0.0
    t_c = flops / (tf * 1e12) * 1e6
    t_l = link_bytes / (NVLINK_GBS_PER_DIR * 1e9) * 1e6
    return {"compute_us": t_c, "link_us": t_l, "roofline_us": max(t_c, t_l), "peaks": pk["source"]}


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
