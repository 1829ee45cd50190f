"""CSV report files in the reference's append-mode convention.

Every invocation appends its header line again followed by its rows
(comm_comp/exp3_gemm_rs_fused.cu:572-580), so a file may hold several headers;
:func:`read_rows` copes with that the way the reference's analyser does
(comm_comp/analyze_rerun.py:32-59).  Column lists below are the reference's
headers verbatim, with this library's extra columns appended at the end.
"""
from __future__ import annotations

import os

EXTRA_COLUMNS = ["max_over_ranks_us", "nccl_cublas_us", "speedup", "roofline_us", "pct_roofline", "dtype"]

# comm_comp/exp3_gemm_rs_fused.cu:575-580
EXP3_FUSED_COLUMNS = ("m,n,k,world,rank,base_us,base_p95,ctrl_us,ctrl_p95,fused_us,fused_p95,struct_sd,comm_sd,"
                      "total_sd,pull_gbps,max_rel_diff,base_p50,ctrl_p50,fused_p50,base_min,ctrl_min,fused_min,"
                      "comm_sd_p50,comm_sd_skew,comm_abs_us,order,iters").split(",") + EXTRA_COLUMNS + ["knobs"]
# comm_comp/exp3_gemm_rs_fused.cu:501 (per-iteration dump, one file per rank)
EXP3_ITER_COLUMNS = "m,n,k,world,rank,variant,iter,us".split(",")
# comm_comp/exp2_ag_gemm_granularity.cu:446-448
EXP2_COLUMNS = ("m,n,k,world,S,chunk_rows,chunk_mib,mode,streams,t_full_us,t_seg_us,t_comm_us,t_ovl_us,seg_eff,"
                "comm_gbps,overlap_eff,e2e_tflops,verify").split(",") + EXTRA_COLUMNS
# comm_comp/exp3_epilogue_remote.cu:256-257
EXP3_EPILOGUE_COLUMNS = ("m,n,k,epi,mode,peer,iter_us,iter_p95,slowdown,tflops,d_write_gbps,verify").split(",") + EXTRA_COLUMNS
# comm_comp/exp1_ce_interference.cu:492-494
EXP1_COLUMNS = ("pattern,m,n,k,msg_bytes,legs,alone_us,ovl_us,alone_p95,ovl_p95,S_c,tflops_alone,tflops_ovl,"
                "comm_alone_gbps,comm_ovl_gbps,gaps").split(",") + EXTRA_COLUMNS
# signalling/signal_fanin.cu:557
SIGNAL_FANIN_COLUMNS = "mode,fanin,bytes,min_us,p50_us,p95_us,p99_us,verify".split(",")
# l2_peer_cache/peer_l2_probe.cu:1365-1375
PEER_L2_BW_COLUMNS = ("build,target,bytes,frac_l2,iters_per_thread,blocks,threads,logical_bytes,ms_med,ms_min,gbps,"
                      "via,dir,tma_tile_bytes").split(",")
PEER_L2_LAT_COLUMNS = "build,target,bytes,frac_l2,lines,hops,ms,ns_per_hop".split(",")
PEER_L2_WIRE_COLUMNS = ("build,target,bytes,launches,iters_per_thread,asked_bytes,ms,gbps,wire_rx_bytes,wire_tx_bytes,"
                        "rx_over_asked,tx_over_asked,idle_rx_bps,idle_tx_bps,counters_ok,via,dir,tma_tile_bytes").split(",")
# tests/interference_matrix.cu:839-841
INTERFERENCE_COLUMNS = ("mode,probe,comm,probe_dev,probe_sms,comm_sms,msg_bytes,comm_alone_gbps,comm_ovl_gbps,S_m,"
                        "probe_alone,probe_ovl,unit,S_c").split(",")
# tests/intra_sm_matrix.cu:621-622
INTRA_SM_COLUMNS = "probe,comm,warps,comm_warps,comm_ctas,msg_bytes,comm_gbps,full,base,ovl,unit,S_warp,S_intra,S_pure".split(",")
# tests/pipeline_e2e.cu:503-504
PIPELINE_E2E_COLUMNS = "method,intensity,flop_per_byte,Tc_src_ms,Tm_ms,Tc_dst_ms,To_ms,pred_ms,err_pct,errors".split(",")
# tests/ce_gemm_overlap.cu:719-722
CE_GEMM_OVERLAP_COLUMNS = ("m,n,k,dtype,comm,dir,msg_bytes,gemm_alone_us,gemm_ovl_us,gemm_alone_p95,gemm_ovl_p95,S_c,"
                           "tflops_alone,tflops_ovl,comm_alone_gbps,comm_ovl_gbps_approx,comm_ovl_gbps,S_m,gaps").split(",")
# The reference prints these three as stdout tables only; the CSV headers follow its table columns
# (tests/pk_bw_sweep.cu:759-761,817-820; tests/p2p_ce_vs_tma.cu:779-780; tests/sync_cost.cu:353-354).
PK_BW_COLUMNS = "figure,mover,msg_bytes,sms,total_bytes,us,gbps,verify".split(",")
P2P_CE_VS_TMA_COLUMNS = "method,tokens,hidden,bytes,avg_us,p50_us,p99_us,gbps,verify".split(",")
SYNC_COST_COLUMNS = "section,variant,payload_bytes,value,unit".split(",")
# End-to-end MLP block (no counterpart in the reference).
MLP_E2E_COLUMNS = ("tokens,hidden,ffn,world,fused_us,fused_p95,ag_us,silu_us,rs_us,nccl_cublas_us,speedup,"
                   "roofline_us,pct_roofline,max_rel_diff,iters,dtype,graph_us").split(",")


class CsvAppender:
    def __init__(self, path: str | None, columns: list[str]):
        self.columns = list(columns)
        self.f = None
        if path:
            os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
            self.f = open(path, "a")
            self.f.write(",".join(self.columns) + "\n")

    def row(self, **kv) -> None:
        if not self.f:
            return
        vals = []
        for c in self.columns:
            v = kv.get(c, "")
            if isinstance(v, float):
                v = f"{v:.4f}" if abs(v) < 100 else f"{v:.2f}"
            vals.append(str(v).replace(",", "|"))
        self.f.write(",".join(vals) + "\n")
        self.f.flush()

    def close(self) -> None:
        if self.f:
            self.f.close()
            self.f = None


def read_rows(path: str) -> list[dict]:
    """Reads a multi-header append-mode CSV: a line that starts with the first
    column name of the current header is taken as a new header."""
    rows, header = [], None
    with open(path) as f:
        for line in f:
            parts = [p.strip() for p in line.rstrip("\n").split(",")]
            if not parts or parts == [""]:
                continue
            if header is None or parts[0] == header[0] or (not _is_number(parts[0]) and parts[0] in ("m", "mode", "bytes", "iter", "pattern", "build", "probe", "method", "figure", "section", "tokens")):
                header = parts
                continue
            rows.append({h: (parts[i] if i < len(parts) else "") for i, h in enumerate(header)})
    return rows


def _is_number(s: str) -> bool:
    try:
        float(s)
        return True
    except ValueError:
        return False
