"""tcgen05 GEMM kernels vs a plain PyTorch fp32 reference (single GPU)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(A, Bt):
    return A.float() @ Bt.float().t()


def _rel(out, ref):
    return ((out.float() - ref).abs() / (ref.abs() + 1)).max().item()


@pytest.mark.parametrize("cta_group", [1, 2])
@pytest.mark.parametrize("shape", [(256, 256, 64), (512, 768, 320), (1024, 512, 1024), (2048, 2304, 512)])
def test_plain_gemm_matches_fp32(native_lib, cta_group, shape):
    from tileccl_b200.ops.gemm import GemmPlan
    M, N, K = shape
    torch.manual_seed(M + N + K)
    A = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    Bt = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    plan = GemmPlan(A, Bt, cta_group=cta_group, timeout_ms=1000)
    out = plan()
    plan.check()
    assert _rel(out, _ref(A, Bt)) < 1e-2
    # a second call of the same plan gives the same bits
    first = out.clone()
    plan()
    plan.check()
    assert torch.equal(first, plan.out)


def test_plain_gemm_strided_operands(native_lib):
    from tileccl_b200.ops.gemm import GemmPlan
    torch.manual_seed(3)
    big_a = torch.randn(512, 1024, device="cuda", dtype=torch.bfloat16)
    big_b = torch.randn(512, 1024, device="cuda", dtype=torch.bfloat16)
    A, Bt = big_a[:, 256:768], big_b[:, :512]     # row pitch 1024, K = 512
    out_big = torch.zeros(512, 1024, device="cuda", dtype=torch.bfloat16)
    out = out_big[:, 512:]
    plan = GemmPlan(A, Bt, out=out, cta_group=2, timeout_ms=1000)
    plan()
    plan.check()
    assert _rel(out, _ref(A, Bt)) < 1e-2
    assert out_big[:, :512].abs().max().item() == 0


def test_plan_rejects_bad_shapes(native_lib):
    from tileccl_b200.ops.gemm import GemmPlan
    A = torch.randn(200, 64, device="cuda", dtype=torch.bfloat16)
    Bt = torch.randn(256, 64, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        GemmPlan(A, Bt, cta_group=1)


@pytest.mark.parametrize("cta_group", [1, 2])
def test_gemm_rs_world1_reduces_its_own_partials(native_lib, cta_group):
    """World of one: nothing to reduce, the epilogue writes the shard itself (the staged path with the
    signalling and reduce warps is forced in test_gemm_rs_world1_32_byte_stores)."""
    from tileccl_b200.ops.gemm_rs import GemmRs
    from tileccl_b200.parallel.heap import SymmetricHeap
    torch.manual_seed(5)
    M, N, K = 1024, 512, 384
    heap = SymmetricHeap(64 << 20)
    A = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    Bt = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    op = GemmRs(heap, A, Bt, cta_group=cta_group, timeout_ms=1000)
    for _ in range(3):                      # epochs advance, counters are never reset
        out = op()
        op.check()
        assert _rel(out, _ref(A, Bt)) < 1e-2
        op.stage.fill_(float("nan"))        # stale staging must not leak into the next call
    heap.close()


@pytest.mark.parametrize("cta_group", [1, 2])
def test_gemm_rs_world1_32_byte_stores(native_lib, cta_group):
    """The opt-in epilogue with st.global.v8.b32 gives the same bits as the 16-byte one."""
    from tileccl_b200.ops.gemm_rs import GemmRs
    from tileccl_b200.parallel.heap import SymmetricHeap
    torch.manual_seed(11)
    M, N, K = 512, 768, 192
    heap = SymmetricHeap(64 << 20)
    A = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    Bt = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    ref_op = GemmRs(heap, A, Bt, cta_group=cta_group, force_staged=True, timeout_ms=1000)
    op = GemmRs(heap, A, Bt, cta_group=cta_group, force_staged=True, timeout_ms=1000, st256=True)
    op.stage.fill_(float("nan"))
    want = ref_op().clone()
    ref_op.check()
    got = op()
    op.check()
    assert torch.equal(got, want)
    assert _rel(got, _ref(A, Bt)) < 1e-2
    heap.close()


@pytest.mark.parametrize("cta_group", [1, 2])
def test_plain_gemm_32_byte_stores(native_lib, cta_group):
    from tileccl_b200.ops.gemm import GemmPlan
    torch.manual_seed(12)
    A = torch.randn(512, 320, device="cuda", dtype=torch.bfloat16)
    Bt = torch.randn(768, 320, device="cuda", dtype=torch.bfloat16)
    want = GemmPlan(A, Bt, cta_group=cta_group, timeout_ms=1000)().clone()
    plan = GemmPlan(A, Bt, cta_group=cta_group, timeout_ms=1000, store="st256")
    got = plan()
    plan.check()
    assert torch.equal(got, want)


@pytest.mark.parametrize("cta_group", [1, 2])
def test_plain_gemm_tma_store_epilogue(native_lib, cta_group):
    """cp.async.bulk.tensor stores from the staging buffer give the same bits as st.global, also with row
    segments routed to separate buffers."""
    from tileccl_b200.ops.gemm import GemmPlan
    torch.manual_seed(13)
    M, N, K = 1024, 768, 320
    A = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    Bt = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    want = GemmPlan(A, Bt, cta_group=cta_group, timeout_ms=1000)().clone()
    plan = GemmPlan(A, Bt, cta_group=cta_group, timeout_ms=1000, store="tma")
    got = plan()
    plan.check()
    assert torch.equal(got, want)
    parts = [torch.full((M // 2, N), float("nan"), device="cuda", dtype=torch.bfloat16) for _ in range(2)]
    seg = GemmPlan(A, Bt, cta_group=cta_group, timeout_ms=1000, store="tma", seg_rows=M // 2, dst_ptrs=[t.data_ptr() for t in parts])
    seg()
    seg.check()
    assert torch.equal(torch.cat(parts, 0), want)


def test_ag_gemm_world1(native_lib):
    from tileccl_b200.ops.ag_gemm import AgGemm
    from tileccl_b200.parallel.heap import SymmetricHeap
    torch.manual_seed(6)
    M, N, K = 512, 768, 256
    heap = SymmetricHeap(64 << 20)
    Bt = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    op = AgGemm(heap, M, K, Bt, cta_group=2, timeout_ms=1000)
    op.a_shard.copy_(torch.randn(M, K, device="cuda", dtype=torch.bfloat16))
    out = op()
    op.check()
    assert _rel(out, _ref(op.a_full, Bt)) < 1e-2
    heap.close()


def test_wait_runs_out_and_reports_status(native_lib):
    """A fused GEMM+RS whose counters can never reach the target (the plan is
    told the world is 2 but only this rank ever signals) must come back with a
    status word instead of hanging; the context stays usable."""
    from tileccl_b200 import _native
    from tileccl_b200.ops._plan import KernelTimeout, Plan
    from tileccl_b200.parallel.heap import SymmetricHeap
    heap = SymmetricHeap(64 << 20)
    M, N, K = 512, 256, 64
    A = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    Bt = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    stage = heap.empty((2, M // 2, N))
    cnt = heap.zeros((2, (M // 2 // 128) * (N // 256)))
    bar = heap.zeros((2, 32))
    out = heap.empty((M // 2, N))
    d = _native.GemmDesc()
    d.mode, d.cta_group = _native.MODE_GEMM_RS, 1
    d.M, d.N, d.K, d.lda, d.ldb, d.ldc = M, N, K, K, K, N
    d.A, d.B = A.data_ptr(), Bt.data_ptr()
    d.world, d.rank, d.seg_rows, d.comm_enabled = 2, 0, M // 2, 1
    for s in range(2):                      # "rank 1" is a second set of buffers on this GPU
        d.dst_base[s] = stage.data_ptr()
        d.dst_row_off[s] = 0
        d.rs_tile_cnt[s] = cnt[s].data_ptr()
        d.barrier[s] = bar[s].data_ptr()
    d.rs_stage, d.rs_out, d.ld_out, d.rs_chunks = stage.data_ptr(), out.data_ptr(), N, 1
    d.timeout_ns = 200_000_000              # 0.2 s
    plan = Plan(d)
    plan.run()
    with pytest.raises(KernelTimeout) as ei:
        plan.check()
    assert ei.value.code in (5, 6)          # the start barrier or a tile counter, whichever gave up first
    # the device still works
    x = torch.ones(8, device="cuda")
    assert float((x * 2).sum()) == 16.0
    heap.close()


def test_elementwise_kernels(native_lib):
    from tileccl_b200.ops import elementwise as ew
    torch.manual_seed(7)
    gu = torch.randn(300, 512, device="cuda", dtype=torch.bfloat16)
    out = ew.silu_mul(gu)
    g, u = gu[:, :256].float(), gu[:, 256:].float()
    ref = torch.nn.functional.silu(g) * u
    assert ((out.float() - ref).abs() / (ref.abs() + 1)).max().item() < 1e-2

    t = torch.empty(1 << 20, device="cuda", dtype=torch.bfloat16)
    ew.fill_normal_(t, seed=1234)
    t2 = torch.empty_like(t)
    ew.fill_normal_(t2, seed=1234)
    assert torch.equal(t, t2)
    f = t.float()
    assert abs(f.mean().item()) < 5e-3 and abs(f.std().item() - 1.0) < 1e-2

    ref32 = torch.randn(5000, device="cuda")
    got = (ref32 + 0.01).bfloat16()
    want = ((got.float() - ref32).abs() / (ref32.abs() + 1)).max().item()
    assert abs(ew.max_rel_err(got, ref32) - want) < 1e-6


@pytest.mark.parametrize("cta_group", [1, 2])
def test_fused_silu_mul_epilogue(native_lib, cta_group):
    """silu(x @ Wg.T) * (x @ Wu.T) straight from the accumulators, gate/up rows interleaved per tile."""
    from tileccl_b200.ops.gemm import GemmPlan, deinterleave_gate_up, interleave_gate_up
    torch.manual_seed(9)
    M, F, K = 512, 384, 320
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    wg = torch.randn(F, K, device="cuda", dtype=torch.bfloat16) * 0.1
    wu = torch.randn(F, K, device="cuda", dtype=torch.bfloat16) * 0.1
    w = interleave_gate_up(wg, wu)
    g2, u2 = deinterleave_gate_up(w)
    assert torch.equal(g2, wg) and torch.equal(u2, wu)
    plan = GemmPlan(x, w, cta_group=cta_group, epi="silu_mul", timeout_ms=1000)
    out = plan()
    plan.check()
    assert out.shape == (M, F)
    ref = torch.nn.functional.silu(x.float() @ wg.float().t()) * (x.float() @ wu.float().t())
    assert _rel(out, ref) < 1e-2


def test_torch_op_layer_single_gpu(native_lib):
    """torch.ops.tileccl.* on one GPU (world of one): plans are cached per operand set."""
    import tileccl_b200 as tc
    torch.manual_seed(21)
    A = torch.randn(512, 384, device="cuda", dtype=torch.bfloat16)
    Bt = torch.randn(768, 384, device="cuda", dtype=torch.bfloat16)
    ref = _ref(A, Bt)
    tc.init(128 << 20)
    try:
        assert _rel(torch.ops.tileccl.gemm(A, Bt), ref) < 1e-2
        assert _rel(torch.ops.tileccl.gemm_rs(A, Bt), ref) < 1e-2
        y1 = torch.ops.tileccl.ag_gemm(A, Bt)
        assert _rel(y1, ref) < 1e-2
        A2 = torch.randn_like(A)
        y2 = torch.ops.tileccl.ag_gemm(A2, Bt)            # same plan, new shard contents
        assert y2.data_ptr() == y1.data_ptr() and _rel(y2, _ref(A2, Bt)) < 1e-2
        gu = torch.randn(256, 512, device="cuda", dtype=torch.bfloat16)
        g, u = gu[:, :256].float(), gu[:, 256:].float()
        assert _rel(torch.ops.tileccl.silu_mul(gu), torch.nn.functional.silu(g) * u) < 2e-2
        torch.ops.tileccl.barrier()
        tc.check_all()
    finally:
        tc.shutdown()


def test_fused_ops_replay_from_a_cuda_graph(native_lib):
    """With the call number kept in device memory the fused kernels can be captured once and replayed:
    epochs advance on the device, counters are never reset, results stay right."""
    from tileccl_b200.ops._plan import capture_graph
    from tileccl_b200.ops.ag_gemm import AgGemm
    from tileccl_b200.ops.gemm_rs import GemmRs
    from tileccl_b200.parallel.heap import SymmetricHeap
    torch.manual_seed(31)
    M, N, K = 1024, 512, 384
    heap = SymmetricHeap(64 << 20)
    A = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    Bt = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    rs = GemmRs(heap, A, Bt, cta_group=2, force_staged=True, timeout_ms=1000, device_epoch=True)
    ag = AgGemm(heap, M, K, Bt, cta_group=2, timeout_ms=1000, device_epoch=True)
    ag.a_shard.copy_(A)

    def both():
        rs()
        ag()

    g = capture_graph(both, warmup=2)                 # 2 eager calls; capturing itself runs nothing
    torch.cuda.synchronize()
    assert rs.plan.epoch == 2 and ag.plan.epoch == 2
    for i in range(3):
        rs.out.fill_(float("nan"))
        rs.stage.fill_(float("nan"))
        ag.out.fill_(float("nan"))
        g.replay()
        torch.cuda.synchronize()
        rs.check()
        ag.check()
        assert _rel(rs.out, _ref(A, Bt)) < 1e-2 and _rel(ag.out, _ref(A, Bt)) < 1e-2
        assert rs.plan.epoch == 3 + i
        rs.audit()
    heap.close()


@pytest.mark.parametrize("cta_group", [1, 2])
def test_gemm_rs_publishes_a_tile_only_after_all_four_warps_stored_it(native_lib, cta_group):
    """One epilogue warp is made to lag by several microseconds per tile (after it has handed the accumulator
    back), so the other three run a tile or two ahead.  The staging buffer is poisoned with NaN before every
    call: if a tile were published to the reduce warps before the slow warp's 32 rows are stored, NaNs (or the
    previous call's rows) would reach the output.  Many tiles per CTA, so that the lead builds up."""
    from tileccl_b200.ops.gemm_rs import GemmRs
    from tileccl_b200.parallel.heap import SymmetricHeap
    torch.manual_seed(41)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    M, N, K = 128 * cta_group * 8, 256 * (sms // cta_group), 128      # 8 tiles per CTA (or CTA pair), short mainloop
    heap = SymmetricHeap(2 * M * N * 2 + (16 << 20))
    A = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    Bt = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    ref = _ref(A, Bt)
    op = GemmRs(heap, A, Bt, cta_group=cta_group, force_staged=True, timeout_ms=2000, ablate=8)
    for _ in range(3):
        op.stage.fill_(float("nan"))
        op.out.fill_(float("nan"))
        out = op()
        op.check()
        assert not torch.isnan(out).any()
        assert _rel(out, ref) < 1e-2
    heap.close()


def test_plan_set_operands_repoints_a_cached_plan(native_lib):
    """A plan re-pointed at new operands of the same layout reads the new ones and keeps no reference."""
    import gc
    import weakref
    from tileccl_b200.ops.gemm import GemmPlan
    torch.manual_seed(43)
    A = torch.randn(512, 256, device="cuda", dtype=torch.bfloat16)
    Bt = torch.randn(512, 256, device="cuda", dtype=torch.bfloat16)
    plan = GemmPlan(A, Bt, cta_group=2, timeout_ms=1000, hold_operands=False)
    assert _rel(plan(), _ref(A, Bt)) < 1e-2
    wr = weakref.ref(A)
    A2 = torch.randn_like(A)
    B2 = torch.randn_like(Bt)
    plan.set_operands(A2, B2)
    del A
    gc.collect()
    assert wr() is None                       # the plan did not keep the first activation alive
    assert _rel(plan(), _ref(A2, B2)) < 1e-2
    plan.check()
    with pytest.raises(ValueError):
        plan.set_operands(A2[:256], B2)


def test_torch_ops_reuse_one_plan_for_fresh_activations(native_lib):
    """A loop that allocates a new activation every step must reuse one plan (and one staging buffer): the
    symmetric heap's cursor does not move after the first call."""
    import tileccl_b200 as tc
    torch.manual_seed(44)
    Bt = torch.randn(512, 384, device="cuda", dtype=torch.bfloat16)
    h = tc.init(128 << 20)
    try:
        keep = []
        cursor = None
        for i in range(6):
            A = torch.randn(512, 384, device="cuda", dtype=torch.bfloat16)
            keep.append(A)                    # keeps every address distinct
            y = torch.ops.tileccl.gemm_rs(A, Bt)
            assert _rel(y, _ref(A, Bt)) < 1e-2
            z = torch.ops.tileccl.gemm(A, Bt)
            assert _rel(z, _ref(A, Bt)) < 1e-2
            if i == 0:
                cursor = h._cursor
            assert h._cursor == cursor
        tc.check_all()
    finally:
        tc.shutdown()
