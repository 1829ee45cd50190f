"""Tensor-parallel gated-SiLU MLP block (Llama-3-70B shaped by default),
sequence-sharded activations in and out:

    x_shard [T/tp, H] --AG+GEMM(gate|up)--> [T, 2F/tp] --SiLU*mul--> [T, F/tp]
                      --GEMM+RS(down)----> y_shard [T/tp, H]

Two kernel launches per forward: the all-gather GEMM, whose epilogue applies
SiLU(gate) * up on the accumulators (gate and up rows of the weight are
interleaved in 128-row blocks so that every output tile holds matching
columns), and the GEMM reduce-scatter.  ``fuse_silu=False`` keeps the
stand-alone SiLU*mul kernel between them (three launches).  The reference has no model; this is
the end-to-end pipeline named by the benchmark configuration (hidden 8192, ffn
28672, 16384 tokens, tp = 8).
"""
from __future__ import annotations

import torch

from ..ops import elementwise as ew
from ..ops.ag_gemm import AgGemm
from ..ops.gemm_rs import GemmRs
from ..parallel.heap import SymmetricHeap


def heap_bytes(tokens: int, hidden: int, ffn: int, world: int) -> int:
    """Symmetric-heap bytes one :class:`TpMlp` takes per rank."""
    f = ffn // world
    return (tokens * hidden * 2            # gathered x
            + tokens * hidden * 2          # RS staging
            + tokens // world * hidden * 2 # RS output
            + (4 << 20))


class TpMlp:
    def __init__(self, heap: SymmetricHeap, tokens: int, hidden: int = 8192, ffn: int = 28672,
                 cta_group: int = 2, gather_rows: int = 512, seed: int = 0, init_std: float = 0.02,
                 fuse_silu: bool = True, graph: bool = False, num_ctas: int = 0):
        """``num_ctas`` caps the grid of both kernels (0 = one CTA per SM): the all-gather GEMM needs all its
        CTAs resident at once, so a caller that runs other kernels beside the block leaves them SMs this way."""
        world, rank = heap.world, heap.rank
        if ffn % world or tokens % world:
            raise ValueError("ffn and tokens must be divisible by the world size")
        f = ffn // world
        self.tokens, self.hidden, self.ffn_local = tokens, hidden, f
        dev = torch.device("cuda", torch.cuda.current_device())
        # Weights in the K-major layout the kernels take: [out_features, in_features].
        # w_gate_up rows: fuse_silu -> 128 gate rows, 128 up rows, 128 gate rows, ... (interleave_gate_up);
        # otherwise all gate rows, then all up rows.
        self.fuse_silu = fuse_silu and f % 128 == 0
        self.w_gate_up = torch.empty(2 * f, hidden, dtype=torch.bfloat16, device=dev)
        self.w_down = torch.empty(hidden, f, dtype=torch.bfloat16, device=dev)
        ew.fill_normal_(self.w_gate_up, seed=seed * 1000 + 2 * rank, std=init_std)
        ew.fill_normal_(self.w_down, seed=seed * 1000 + 2 * rank + 1, std=init_std)
        self.act = torch.empty(tokens, f, dtype=torch.bfloat16, device=dev)
        if self.fuse_silu:
            self.h = None
            self.ag = AgGemm(heap, tokens, hidden, self.w_gate_up, cta_group=cta_group,
                             gather_rows=gather_rows, out=self.act, epi="silu_mul", device_epoch=graph, num_ctas=num_ctas)
        else:
            self.h = torch.empty(tokens, 2 * f, dtype=torch.bfloat16, device=dev)
            self.ag = AgGemm(heap, tokens, hidden, self.w_gate_up, cta_group=cta_group,
                             gather_rows=gather_rows, out=self.h, device_epoch=graph, num_ctas=num_ctas)
        self.rs = GemmRs(heap, self.act, self.w_down, cta_group=cta_group, device_epoch=graph, num_ctas=num_ctas)
        self._graph = None
        self._want_graph = graph

    @property
    def x_shard(self) -> torch.Tensor:
        """This rank's [T/tp, H] input slot inside the gathered buffer; write the input here."""
        return self.ag.a_shard

    def forward(self, stream=None) -> torch.Tensor:
        self.ag(stream)
        if not self.fuse_silu:
            ew.silu_mul(self.h, self.act, stream)
        return self.rs(stream)

    __call__ = forward

    def capture(self, warmup: int = 2):
        """Captures the block (two or three launches) in a CUDA graph; needs ``graph=True`` at construction
        so that the kernels keep their call numbers in device memory.  ``replay()`` then runs the block with
        one launch from the host and returns the output buffer.  Collective: every rank captures and replays
        in step."""
        if not self._want_graph:
            raise RuntimeError("build the block with graph=True to capture it")
        from ..ops._plan import capture_graph
        self._graph = capture_graph(self.forward, warmup)
        return self._graph

    def replay(self) -> torch.Tensor:
        if self._graph is None:
            raise RuntimeError("capture() first")
        self._graph.replay()
        return self.rs.out

    def check(self) -> None:
        self.ag.check()
        self.rs.check()

    def gate_up_plain(self) -> torch.Tensor:
        """The gate|up weight in the plain layout (all gate rows, then all up rows)."""
        if not self.fuse_silu:
            return self.w_gate_up
        from ..ops.gemm import deinterleave_gate_up
        g, u = deinterleave_gate_up(self.w_gate_up)
        return torch.cat([g, u], 0).contiguous()

    @property
    def launches(self) -> int:
        return self.ag.launches + self.rs.launches + (0 if self.fuse_silu else self.ag.launches)
