"""Shared helpers of the op wrappers: plan lifetime, status word, stream."""
from __future__ import annotations

import ctypes as C

import torch

from .. import _native


class KernelTimeout(RuntimeError):
    """A device-side wait ran out; the kernel returned with a status word."""

    def __init__(self, code: int, block: int, d0: int, d1: int):
        self.code, self.block, self.detail = code, block, (d0, d1)
        super().__init__(
            f"tileccl kernel gave up: {_native.status_string(code)} "
            f"(code {code}, block {block}, detail {d0}, {d1})"
        )


class Plan:
    """Owns one native GEMM plan, its status word and its call counter.

    The fused kernels compare flag counters with ``call number x producers``.  By default the call number
    is a host counter passed with every launch.  With ``device_epoch=True`` it lives in device memory and
    the kernel advances it itself, so the launch carries no per-call argument and can be captured in a CUDA
    graph and replayed (:func:`capture_graph`); every rank must then replay the same number of times.
    """

    def __init__(self, desc: _native.GemmDesc, keep_alive=(), device_epoch: bool = False):
        self.lib = _native.lib()
        self.status = torch.zeros(4, dtype=torch.int32, device="cuda")
        desc.status = self.status.data_ptr()
        self.epoch_dev = torch.zeros(2, dtype=torch.int32, device="cuda") if device_epoch else None
        desc.epoch_dev = self.epoch_dev.data_ptr() if device_epoch else None
        err = C.create_string_buffer(256)
        self.handle = self.lib.tcl_gemm_plan_create(C.byref(desc), err, 256)
        if not self.handle:
            raise ValueError(f"tileccl plan rejected: {err.value.decode()}")
        self.desc = desc
        self._host_epoch = 0
        self.launches = 0
        self._keep = keep_alive

    @property
    def epoch(self) -> int:
        """Calls made so far (with a device-side counter: calls completed; reading it synchronises)."""
        if self.epoch_dev is not None:
            return int(self.epoch_dev[0].item())
        return self._host_epoch

    @property
    def grid(self) -> int:
        return self.lib.tcl_gemm_plan_grid(self.handle)

    def run(self, stream: torch.cuda.Stream | None = None) -> None:
        s = stream if stream is not None else torch.cuda.current_stream()
        self._host_epoch += 1
        rc = self.lib.tcl_gemm_plan_run(self.handle, self._host_epoch, C.c_void_p(s.cuda_stream))
        _native.check(rc, "kernel launch")
        self.launches += 1

    def set_operands(self, A: torch.Tensor, Bt: torch.Tensor) -> None:
        """Points the plan at other operands of the same shape and row pitch (host-side re-encoding of the
        two tensor maps, no device work).  The plan keeps no reference to them: the caller keeps them alive
        until the launches that read them have finished."""
        d = self.desc
        if tuple(A.shape) != (d.M, d.K) or A.stride(0) != d.lda or tuple(Bt.shape) != (d.N, d.K) or Bt.stride(0) != d.ldb:
            raise ValueError("set_operands: shape or row pitch differs from the plan's")
        _native.check(self.lib.tcl_gemm_plan_set_operands(self.handle, C.c_void_p(A.data_ptr()), C.c_void_p(Bt.data_ptr())), "set_operands")

    def check(self) -> None:
        """Synchronises and raises :class:`KernelTimeout` if a wait ran out."""
        st = self.status.tolist()
        if st[0] != 0:
            raise KernelTimeout(*st)

    def __del__(self):
        try:
            if getattr(self, "handle", None):
                self.lib.tcl_gemm_plan_destroy(self.handle)
                self.handle = None
        except Exception:
            pass


def require_bf16_rowmajor(t: torch.Tensor, name: str) -> None:
    if t.dtype != torch.bfloat16 or not t.is_cuda or t.dim() != 2 or t.stride(1) != 1:
        raise ValueError(f"{name} must be a 2-D bf16 CUDA tensor with unit inner stride")


def capture_graph(fn, warmup: int = 2) -> torch.cuda.CUDAGraph:
    """Captures one call of ``fn`` (launches of plans built with ``device_epoch=True``, torch ops that do
    not allocate) in a CUDA graph, after ``warmup`` eager calls on a side stream.  ``graph.replay()`` then
    repeats the call with one launch from the host.  On several ranks every rank captures and replays in
    step: the warm-up calls count as calls like any other, capturing runs nothing, each replay is one call."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(warmup):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    return g
