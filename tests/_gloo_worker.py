"""CPU worker (gloo): the host-side collective helpers the GPU drivers rely on."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from tileccl_b200.ops import oracle  # noqa: E402
from tileccl_b200.parallel import group as G  # noqa: E402

import numpy as np  # noqa: E402


def main():
    rank, world, _ = G.init(backend="gloo")
    assert G.world_size() == world and G.rank() == rank
    got = G.all_gather_object({"rank": rank, "blob": bytes([rank]) * 64})
    assert [g["rank"] for g in got] == list(range(world)) and got[-1]["blob"][0] == world - 1
    assert G.max_over_ranks(10.0 + rank) == 10.0 + world - 1
    G.host_barrier()
    # the fused-op semantics on CPU ranks: every rank holds A_r, B_r; gather them and compare the
    # rank's shard of the reduce-scatter oracle with a direct computation
    A, B = oracle.normal_inputs(world, 64 * world, 32, 48, seed=3)
    mine = G.all_gather_object((A[rank], B[rank]))
    shards = oracle.gemm_rs([m[0] for m in mine], [m[1] for m in mine])
    total = sum(a.astype(np.float64) @ b.astype(np.float64) for a, b in zip(A, B))
    np.testing.assert_allclose(shards[rank], total[rank * 64:(rank + 1) * 64], rtol=1e-5, atol=1e-5)
    G.host_barrier()
    G.shutdown()
    if rank == 0:
        print("GLOO_OK")


if __name__ == "__main__":
    main()
