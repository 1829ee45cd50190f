"""Small stand-alone kernels: fused SiLU*mul, N(0,1) fill, verify, device barrier."""
from __future__ import annotations

import ctypes as C

import torch

from .. import _native


def _stream_ptr(stream=None) -> C.c_void_p:
    s = stream if stream is not None else torch.cuda.current_stream()
    return C.c_void_p(s.cuda_stream)


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor | None = None, stream=None) -> torch.Tensor:
    """``silu(gate_up[:, :F]) * gate_up[:, F:]`` for a contiguous bf16 [rows, 2F] input."""
    if gate_up.dtype != torch.bfloat16 or not gate_up.is_contiguous() or gate_up.dim() != 2:
        raise ValueError("gate_up must be a contiguous 2-D bf16 tensor")
    rows, two_f = gate_up.shape
    f = two_f // 2
    if out is None:
        out = torch.empty(rows, f, dtype=torch.bfloat16, device=gate_up.device)
    _native.check(_native.lib().tcl_silu_mul(gate_up.data_ptr(), out.data_ptr(), rows, f, _stream_ptr(stream)), "silu_mul")
    return out


def fill_normal_(t: torch.Tensor, seed: int, mean: float = 0.0, std: float = 1.0, stream=None) -> torch.Tensor:
    """In-place N(mean, std) fill of a contiguous bf16 tensor (counter-based, reproducible)."""
    if t.dtype != torch.bfloat16 or not t.is_contiguous():
        raise ValueError("fill_normal_ wants a contiguous bf16 tensor")
    _native.check(_native.lib().tcl_fill_normal_bf16(t.data_ptr(), t.numel(), seed, mean, std, _stream_ptr(stream)), "fill")
    return t


def max_rel_err(got: torch.Tensor, ref_f32: torch.Tensor, stream=None) -> float:
    """max |got - ref| / (|ref| + 1) computed on the device (bf16 vs fp32 reference)."""
    if got.dtype != torch.bfloat16 or ref_f32.dtype != torch.float32:
        raise ValueError("got must be bf16 and ref fp32")
    got = got.contiguous()
    ref_f32 = ref_f32.contiguous()
    scratch = torch.empty(1024, dtype=torch.float32, device=got.device)
    res = torch.empty(1, dtype=torch.float32, device=got.device)
    _native.check(_native.lib().tcl_max_rel_err(got.data_ptr(), ref_f32.data_ptr(), got.numel(),
                                                scratch.data_ptr(), res.data_ptr(), _stream_ptr(stream)), "verify")
    return float(res.item())


class DeviceBarrier:
    """All-ranks device barrier on a stream (epoch counters, bounded wait).

    ``transport="p2p"``: every rank adds 1 to every rank's counter through the peer mappings (world
    stores per rank).  ``transport="nvls"``: one ``multimem.red.release`` per rank on the counter's
    multicast address, the switch fans it out; needs a heap created with ``multicast=True``.
    """

    def __init__(self, heap, timeout_ms: float = 4000.0, transport: str = "p2p"):
        if transport not in ("p2p", "nvls"):
            raise ValueError(f"unknown barrier transport {transport!r}")
        self.heap = heap
        self.transport = transport
        self.counter = heap.zeros((32,), torch.int32)
        self.status = torch.zeros(4, dtype=torch.int32, device="cuda")
        self.ptrs = (C.c_void_p * _native.MAX_WORLD)(*[heap.peer_ptr(self.counter, r) for r in range(heap.world)])
        self.mc_ptr = heap.mc_ptr(self.counter) if transport == "nvls" else None
        self.epoch = 0
        self.timeout_ns = int(timeout_ms * 1e6)

    def __call__(self, stream=None) -> None:
        self.epoch += 1
        if self.transport == "nvls":
            _native.check(_native.lib().tcl_barrier_all_mc(self.mc_ptr, self.counter.data_ptr(), self.heap.world, self.heap.rank, self.epoch,
                                                           self.status.data_ptr(), self.timeout_ns, _stream_ptr(stream)), "barrier")
            return
        _native.check(_native.lib().tcl_barrier_all(self.ptrs, self.heap.world, self.heap.rank, self.epoch,
                                                    self.status.data_ptr(), self.timeout_ns, _stream_ptr(stream)), "barrier")

    def check(self) -> None:
        st = self.status.tolist()
        if st[0] != 0:
            raise RuntimeError(f"device barrier timed out: rank {st[1]} wanted {st[2]} saw {st[3]}")
