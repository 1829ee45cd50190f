"""CPU oracle of the fused ops, including the world=2 in-process configuration
A[256,512] x B[512,256] fp32 ~ N(0,1) seed 0 -> two [128,256] shards."""
import numpy as np

from tileccl_b200.ops import oracle


def test_gemm_rs_world2_exact_vs_numpy():
    A, B = oracle.normal_inputs(world=2, M=256, N=256, K_local=512, seed=0)
    shards = oracle.gemm_rs(A, B)
    assert len(shards) == 2 and all(s.shape == (128, 256) for s in shards)
    total = A[0].astype(np.float64) @ B[0].astype(np.float64) + A[1].astype(np.float64) @ B[1].astype(np.float64)
    np.testing.assert_array_equal(np.concatenate(shards, axis=0), total.astype(np.float32))


def test_gemm_rs_inputs_are_seeded():
    A1, B1 = oracle.normal_inputs(2, 256, 256, 512, seed=0)
    A2, B2 = oracle.normal_inputs(2, 256, 256, 512, seed=0)
    A3, _ = oracle.normal_inputs(2, 256, 256, 512, seed=1)
    np.testing.assert_array_equal(A1[1], A2[1])
    np.testing.assert_array_equal(B1[0], B2[0])
    assert not np.array_equal(A1[0], A3[0])
    assert abs(float(np.mean(A1[0]))) < 0.02 and abs(float(np.std(A1[0])) - 1.0) < 0.02


def test_ag_gemm_matches_concat():
    rng = np.random.default_rng(1)
    shards = [rng.standard_normal((64, 96)).astype(np.float32) for _ in range(4)]
    Bs = [rng.standard_normal((96, 32)).astype(np.float32) for _ in range(4)]
    outs = oracle.ag_gemm(shards, Bs)
    full = np.concatenate(shards, 0)
    for o, b in zip(outs, Bs):
        np.testing.assert_allclose(o, full @ b, rtol=1e-5, atol=1e-4)


def test_tp_mlp_equals_unsharded():
    rng = np.random.default_rng(2)
    world, T, H, F = 4, 64, 48, 128
    x = rng.standard_normal((T, H)).astype(np.float32)
    wg = rng.standard_normal((H, F)).astype(np.float32) * 0.1
    wu = rng.standard_normal((H, F)).astype(np.float32) * 0.1
    wd = rng.standard_normal((F, H)).astype(np.float32) * 0.1
    g, u = x @ wg, x @ wu
    ref = (g / (1 + np.exp(-g)) * u) @ wd
    fl = F // world
    x_sh = [x[r * T // world:(r + 1) * T // world] for r in range(world)]
    wgu = [np.concatenate([wg[:, r * fl:(r + 1) * fl], wu[:, r * fl:(r + 1) * fl]], axis=1) for r in range(world)]
    wdn = [wd[r * fl:(r + 1) * fl] for r in range(world)]
    outs = oracle.tp_mlp(x_sh, wgu, wdn)
    np.testing.assert_allclose(np.concatenate(outs, 0), ref, rtol=1e-4, atol=1e-4)


def test_max_rel_err_metric():
    ref = np.array([0.0, 1.0, -3.0])
    got = np.array([0.1, 1.0, -2.0])
    assert abs(oracle.max_rel_err(got, ref) - 0.25) < 1e-12
