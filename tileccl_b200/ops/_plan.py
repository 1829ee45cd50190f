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
    """Owns one native GEMM plan, its status word and its call counter."""

    def __init__(self, desc: _native.GemmDesc, keep_alive=()):
        self.lib = _native.lib()
        self.status = torch.zeros(4, dtype=torch.int32, device="cuda")
        desc.status = self.status.data_ptr()
        err = C.create_string_buffer(256)
        self.handle = self.lib.tcl_gemm_plan_create(C.byref(desc), err, 256)
        if not self.handle:
            raise ValueError(f"tileccl plan rejected: {err.value.decode()}")
        self.desc = desc
        self.epoch = 0
        self.launches = 0
        self._keep = keep_alive

    @property
    def grid(self) -> int:
        return self.lib.tcl_gemm_plan_grid(self.handle)

    def run(self, stream: torch.cuda.Stream | None = None) -> None:
        s = stream if stream is not None else torch.cuda.current_stream()
        self.epoch += 1
        rc = self.lib.tcl_gemm_plan_run(self.handle, self.epoch, C.c_void_p(s.cuda_stream))
        _native.check(rc, "kernel launch")
        self.launches += 1

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
