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
from tileccl_b200.ops._plan import KernelTimeout  # noqa: E402
from tileccl_b200.ops.gemm_rs import GemmRs  # noqa: E402
from tileccl_b200.parallel import group as G  # noqa: E402
from tileccl_b200.parallel.heap import SymmetricHeap  # noqa: E402


def rel(out, ref):
    return ((out.float() - ref).abs() / (ref.abs() + 1)).max().item()


def gather(t):
    out = [torch.empty_like(t) for _ in range(dist.get_world_size())]
    dist.all_gather(out, t.contiguous())
    return out


def agree(ok: bool) -> bool:
    """True if every rank says ok (keeps the ranks in lock step after a step that may fail on one of them)."""
    t = torch.tensor([1 if ok else 0], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    return bool(int(t))


def rs_bound(parts, ref, sl, final_ulp=2.0 ** -8):
    """The partials cross NVLink as bf16 and are summed in fp32: every partial and the result are rounded
    once (bf16 unit round-off = 2^-8 relative)."""
    return 1.05 * (2.0 ** -8 * sum(p.abs() for p in parts) + final_ulp * ref.abs())[sl] + 1e-2


def check_gemm_rs(heap, fails, tag, M, N, K, cta_group, iters=3, poison=True, final_ulp=2.0 ** -8, **kw):
    """Fused GEMM+RS against the fp32 sum of the all-gathered partial products.  A time-out on one rank is
    recorded and agreed on by all ranks (nobody raises in the middle of a collective sequence)."""
    rank, world = heap.rank, heap.world
    A = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    Bt = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    op = GemmRs(heap, A, Bt, cta_group=cta_group, timeout_ms=2000, **kw)
    parts = [a.float() @ b.float().t() for a, b in zip(gather(A), gather(Bt))]
    ref = sum(parts)
    seg = M // world
    sl = slice(rank * seg, (rank + 1) * seg)
    bound = rs_bound(parts, ref, sl, final_ulp)
    del parts
    for it in range(iters):
        err = None
        try:
            out = op()
            op.check()
            excess = ((out.float() - ref[sl]).abs() - bound).max().item()
            if not (excess <= 0):
                err = f"error exceeds the bf16 rounding bound by {excess}"
            else:
                op.audit()
        except (KernelTimeout, AssertionError) as e:
            err = str(e)
        if err:
            fails.append(f"gemm_rs {tag} iter {it}: {err}")
        if not agree(err is None):
            return False
        if poison:
            op.stage.fill_(float("nan"))
        torch.cuda.synchronize()
        dist.barrier()
    return True


def check_ag_gemm(heap, fails, tag, M, N, K, cta_group, gather_rows, transport, iters=3, **kw):
    world = heap.world
    Bt = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    op = AgGemm(heap, M, K, Bt, cta_group=cta_group, gather_rows=gather_rows, timeout_ms=2000, transport=transport, **kw)
    for it in range(iters):
        shard = torch.randn(M // world, K, device="cuda", dtype=torch.bfloat16)
        # poison the peers' part of the gathered buffer: stale rows must not be used
        op.a_full.fill_(float("nan"))
        op.a_shard.copy_(shard)
        torch.cuda.synchronize()
        dist.barrier()
        err = None
        try:
            out = op()
            op.check()
        except KernelTimeout as e:
            err = str(e)
        ok = agree(err is None)                  # further collectives only once every rank is known to have come back
        if ok:
            full = torch.cat(gather(shard), 0)
            e = rel(out, full.float() @ Bt.float().t())
            try:
                if not (e <= 2e-2) or not torch.equal(op.a_full, full):
                    err = f"rel err {e}"
                else:
                    op.audit()
            except AssertionError as e2:
                err = str(e2)
            ok = agree(err is None)
        if err:
            fails.append(f"ag_gemm {transport} {tag} rows {gather_rows} iter {it}: {err}")
        if not ok:
            return False
        dist.barrier()
    return True


def nvls_section(fails, world, rank):
    """GEMM + reduce-scatter through the NVSwitch (multimem.ld_reduce) and the multicast barrier.  Every step
    ends with an agreement among the ranks, so a wait that runs out on one rank makes all of them skip the rest
    and take the multicast binding down together, in order; nobody leaves while peers are still bound."""
    from tileccl_b200 import _native
    mc_heap = SymmetricHeap(256 << 20, backend="vmm", multicast=True)
    try:
        # the switch's final conversion is allowed a whole bf16 ulp (2^-7), the partials half an ulp each
        if not check_gemm_rs(mc_heap, fails, "nvls small", 512 * world, 512, 256, 2, iters=2, poison=False, final_ulp=2.0 ** -7, transport="nvls"):
            return
        mc_heap.reset()
        # many tiles per CTA pair, several wraps of the operand stages
        if not check_gemm_rs(mc_heap, fails, "nvls large", 2048 * world, 2048, 1024, 2, iters=2, poison=False, final_ulp=2.0 ** -7, transport="nvls"):
            return
        mc_heap.reset()
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
            bad = any(g < ep for g in got)
            if bad:
                fails.append(f"nvls barrier epoch {ep}: passed before every rank arrived: {got}")
            if not agree(not bad):
                return
        try:
            mbar.check()
        except RuntimeError as e:
            fails.append(str(e))
    finally:
        torch.cuda.synchronize()
        dist.barrier()
        mc_heap.close()


def main():
    rank, world, _ = G.init()
    torch.manual_seed(100 + rank)
    heap = SymmetricHeap(1 << 30)
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
    mark = heap._cursor

    ok = True
    for cta_group in (1, 2):
        if not ok:
            break
        # ---- small shapes: a couple of tiles per CTA ----
        ok = check_gemm_rs(heap, fails, f"g{cta_group}", 256 * cta_group * world * 2, 512, 320, cta_group)
        for gather_rows, transport in ((128, "push"), (256 * cta_group, "push"), (256 * cta_group, "pull")):
            ok = ok and check_ag_gemm(heap, fails, f"g{cta_group}", 256 * cta_group * world, 768, 512, cta_group, gather_rows, transport)
        torch.cuda.synchronize()
        dist.barrier()
        heap._cursor = mark
        # ---- large shapes: every CTA (pair) walks about seven tiles, the operand stages wrap five times per tile,
        # both accumulator buffers and every phase bit are exercised across ranks ----
        Ml = 1024 * world if world * 1024 >= 8192 else 8192
        ok = ok and check_gemm_rs(heap, fails, f"g{cta_group} large", Ml, 4096, 2048, cta_group, iters=2)
        heap._cursor = mark
        # the same with one epilogue warp lagging: a tile must not be announced before all four warps stored it
        ok = ok and check_gemm_rs(heap, fails, f"g{cta_group} large, lagging warp", Ml, 4096, 256, cta_group, iters=2, ablate=8)
        heap._cursor = mark
        for transport in ("pull", "push"):
            ok = ok and check_ag_gemm(heap, fails, f"g{cta_group} large", Ml, 4096, 2048, cta_group, 512, transport, iters=2)
            torch.cuda.synchronize()
            dist.barrier()
            heap._cursor = mark
        # knobs: one fence per tile / per 16 tiles in the signalling warp; two gather warps moving 32 bytes per instruction
        for sb in (1, 16):
            ok = ok and check_gemm_rs(heap, fails, f"g{cta_group} large, signal batch {sb}", Ml, 4096, 512, cta_group, iters=2, signal_batch=sb)
            heap._cursor = mark
        ok = ok and check_ag_gemm(heap, fails, f"g{cta_group} large, 2 gather warps, 32-byte moves", Ml, 4096, 1024, cta_group, 1024, "pull", iters=2,
                                  gather_warps=2, vec32=True)
        torch.cuda.synchronize()
        dist.barrier()
        heap._cursor = mark

    # ---- through the NVSwitch, when multicast is available ----
    from tileccl_b200 import _native
    if ok and _native.lib().tcl_multicast_supported(torch.cuda.current_device()):
        nvls_section(fails, world, rank)

    # ---- torch.ops layer with a fresh activation every call: one plan, the same heap offsets on every rank ----
    if ok:
        import tileccl_b200 as tc
        h2 = tc.init(256 << 20)
        w = torch.randn(512, 256, device="cuda", dtype=torch.bfloat16)
        keep = []
        for it in range(4):
            a = torch.randn(512 * world, 256, device="cuda", dtype=torch.bfloat16)
            if rank % 2 == it % 2:
                keep.append(torch.empty(1 << 20, device="cuda"))   # ranks see different allocator addresses
            keep.append(a)
            y = torch.ops.tileccl.gemm_rs(a, w)
            err = None
            try:
                tc.check_all()
            except KernelTimeout as e:
                err = str(e)
            if agree(err is None):
                parts = [x.float() @ b.float().t() for x, b in zip(gather(a), gather(w))]
                ref = sum(parts)
                seg = a.shape[0] // world
                sl = slice(rank * seg, (rank + 1) * seg)
                excess = ((y.float() - ref[sl]).abs() - rs_bound(parts, ref, sl)).max().item()
                if not (excess <= 0):
                    err = f"error exceeds the bound by {excess}"
                if it == 0:
                    cursor = h2._cursor
                elif h2._cursor != cursor:
                    err = "the plan cache allocated again for a new activation address"
            if err:
                fails.append(f"torch.ops gemm_rs, fresh activation {it}: {err}")
            if not agree(err is None):
                break
        torch.cuda.synchronize()
        dist.barrier()
        tc.shutdown()

    # ---- MLP block ----
    heap._cursor = mark
    tokens, hidden, ffn = 512 * world, 512, 1024 * world
    mlp = TpMlp(heap, tokens, hidden, ffn, cta_group=2, gather_rows=256)
    x = torch.randn(tokens // world, hidden, device="cuda", dtype=torch.bfloat16)
    mlp.x_shard.copy_(x)
    torch.cuda.synchronize()
    dist.barrier()
    y = mlp()
    try:
        mlp.check()
    except KernelTimeout as e:
        fails.append(f"tp_mlp: {e}")
    xf = torch.cat(gather(x), 0).float()
    f = ffn // world
    parts = []
    for wgu, wd in zip(gather(mlp.gate_up_plain()), gather(mlp.w_down)):
        h = xf @ wgu.float().t()                      # the fused epilogue applies SiLU*mul on the fp32 accumulators
        a = (torch.nn.functional.silu(h[:, :f]) * h[:, f:]).bfloat16().float()
        parts.append(a @ wd.float().t())
    ref = sum(parts)[rank * (tokens // world):(rank + 1) * (tokens // world)]
    e = rel(y, ref)
    if not (e <= 2e-2):
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
