"""Worker of the multi-GPU tests: run as one process per GPU by torchrun.

Each check compares a fused op against a plain PyTorch fp32 computation on the
all-gathered inputs.  Prints ``WORKER_OK`` on rank 0 when every check passed.
"""
import ctypes as C
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from tileccl_b200.models.tp_mlp import TpMlp  # noqa: E402
from tileccl_b200.ops import elementwise as ew  # noqa: E402
from tileccl_b200.ops.ag_gemm import AgGemm  # noqa: E402
from tileccl_b200.ops.gemm_rs import GemmRs  # noqa: E402
from tileccl_b200.parallel import group as G  # noqa: E402
from tileccl_b200.parallel.heap import SymmetricHeap  # noqa: E402


def rel(out, ref):
    return ((out.float() - ref).abs() / (ref.abs() + 1)).max().item()


def gather(t):
    out = [torch.empty_like(t) for _ in range(dist.get_world_size())]
    dist.all_gather(out, t.contiguous())
    return out


def main():
    rank, world, _ = G.init()
    torch.manual_seed(100 + rank)
    heap = SymmetricHeap(512 << 20)
    fails = []

    # heap symmetry: a peer's view of a tensor shows what that peer wrote
    t = heap.empty((1024,), torch.int32)
    t.fill_(rank + 1)
    torch.cuda.synchronize()
    dist.barrier()
    for r in range(world):
        v = heap.peer_tensor(t, r)
        if int(v[0]) != r + 1 or int(v[-1]) != r + 1:
            fails.append(f"heap view of rank {r} wrong")
    dist.barrier()

    # device barrier epochs
    bar = ew.DeviceBarrier(heap, timeout_ms=2000)
    for _ in range(5):
        bar()
    torch.cuda.synchronize()
    bar.check()

    for cta_group in (1, 2):
        # ---- fused GEMM + reduce-scatter ----
        M, N, K = 256 * cta_group * world * 2, 512, 320
        A = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        Bt = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
        op = GemmRs(heap, A, Bt, cta_group=cta_group, timeout_ms=2000)
        As, Bs = gather(A), gather(Bt)
        parts = [a.float() @ b.float().t() for a, b in zip(As, Bs)]
        ref = sum(parts)
        seg = M // world
        sl = slice(rank * seg, (rank + 1) * seg)
        # The partials cross NVLink as bf16 and are summed in fp32: every
        # partial and the result are rounded once (bf16 unit round-off = 2^-8 relative).
        bound = 2.0 ** -8 * 1.05 * (sum(p.abs() for p in parts) + ref.abs())[sl] + 1e-2
        for it in range(3):
            out = op()
            op.check()
            excess = ((out.float() - ref[sl]).abs() - bound).max().item()
            if excess > 0:
                fails.append(f"gemm_rs g{cta_group} iter {it}: error exceeds the bf16 rounding bound by {excess}")
            op.audit()
            op.stage.fill_(float("nan"))
            torch.cuda.synchronize()
            dist.barrier()

        # ---- fused all-gather + GEMM ----
        M, N, K = 256 * cta_group * world, 768, 512
        Bt = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
        for gather_rows, transport in ((128, "push"), (256 * cta_group, "push"), (256 * cta_group, "pull")):
            op = AgGemm(heap, M, K, Bt, cta_group=cta_group, gather_rows=gather_rows, timeout_ms=2000, transport=transport)
            for it in range(3):
                shard = torch.randn(M // world, K, device="cuda", dtype=torch.bfloat16)
                # poison the peers' part of the gathered buffer: stale rows must not be used
                op.a_full.fill_(float("nan"))
                op.a_shard.copy_(shard)
                torch.cuda.synchronize()
                dist.barrier()
                out = op()
                op.check()
                full = torch.cat(gather(shard), 0)
                e = rel(out, full.float() @ Bt.float().t())
                if e > 2e-2 or not torch.equal(op.a_full, full):
                    fails.append(f"ag_gemm {transport} g{cta_group} rows {gather_rows} iter {it}: rel err {e}")
                op.audit()
                dist.barrier()

    # ---- GEMM + reduce-scatter through the NVSwitch (multimem.ld_reduce), when multicast is available ----
    from tileccl_b200 import _native
    if _native.lib().tcl_multicast_supported(torch.cuda.current_device()):
        mc_heap = SymmetricHeap(128 << 20, backend="vmm", multicast=True)
        M, N, K = 512 * world, 512, 256
        A = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        Bt = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
        op = GemmRs(mc_heap, A, Bt, cta_group=2, transport="nvls", timeout_ms=2000)
        parts = [a.float() @ b.float().t() for a, b in zip(gather(A), gather(Bt))]
        ref = sum(parts)
        seg = M // world
        sl = slice(rank * seg, (rank + 1) * seg)
        # the switch's final conversion is allowed a whole bf16 ulp (2^-7), the partials half an ulp each
        bound = 1.05 * (2.0 ** -8 * sum(p.abs() for p in parts) + 2.0 ** -7 * ref.abs())[sl] + 1e-2
        for it in range(2):
            out = op()
            op.check()
            excess = ((out.float() - ref[sl]).abs() - bound).max().item()
            if excess > 0:
                fails.append(f"gemm_rs nvls iter {it}: error exceeds the bf16 rounding bound by {excess}")
            op.audit()
            torch.cuda.synchronize()
            dist.barrier()
        del op
        # barrier with one multimem.red per rank: a rank may pass only after every rank arrived
        mbar = ew.DeviceBarrier(mc_heap, timeout_ms=2000, transport="nvls")
        seen = mc_heap.zeros((4 * world,), torch.int32)   # one 16-byte slot per source rank
        mine = torch.zeros(4, dtype=torch.int32, device="cuda")
        lib, vp = _native.lib(), C.c_void_p
        for ep in range(1, 4):
            mine.fill_(ep)
            for r in range(world):   # publish "arrived at ep" on every peer (own copy kernel), then the barrier
                _native.check(lib.tcl_p2p_copy(vp(mc_heap.peer_ptr(seen, r) + 16 * rank), vp(mine.data_ptr()), 16, 1,
                                               vp(torch.cuda.current_stream().cuda_stream)), "p2p_copy")
            mbar()
            torch.cuda.synchronize()
            got = seen[::4].tolist()
            if any(g < ep for g in got):
                fails.append(f"nvls barrier epoch {ep}: passed before every rank arrived: {got}")
        mbar.check()
        dist.barrier()
        mc_heap.close()

    # ---- MLP block ----
    tokens, hidden, ffn = 512 * world, 512, 1024 * world
    mlp = TpMlp(heap, tokens, hidden, ffn, cta_group=2, gather_rows=256)
    x = torch.randn(tokens // world, hidden, device="cuda", dtype=torch.bfloat16)
    mlp.x_shard.copy_(x)
    torch.cuda.synchronize()
    dist.barrier()
    y = mlp()
    mlp.check()
    xf = torch.cat(gather(x), 0).float()
    f = ffn // world
    parts = []
    for wgu, wd in zip(gather(mlp.gate_up_plain()), gather(mlp.w_down)):
        h = xf @ wgu.float().t()                      # the fused epilogue applies SiLU*mul on the fp32 accumulators
        a = (torch.nn.functional.silu(h[:, :f]) * h[:, f:]).bfloat16().float()
        parts.append(a @ wd.float().t())
    ref = sum(parts)[rank * (tokens // world):(rank + 1) * (tokens // world)]
    e = rel(y, ref)
    if e > 2e-2:
        fails.append(f"tp_mlp rel err {e}")

    flag = torch.tensor([len(fails)], device="cuda")
    dist.all_reduce(flag)
    if fails:
        print(f"[rank {rank}] FAILURES: {fails}", flush=True)
    torch.cuda.synchronize()
    dist.barrier()
    heap.close()
    if rank == 0 and int(flag) == 0:
        print("WORKER_OK", flush=True)
    G.shutdown()
    sys.exit(1 if int(flag) else 0)


if __name__ == "__main__":
    main()
