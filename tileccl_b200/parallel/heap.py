"""Symmetric heap: the same byte offset names the same object on every rank.

Each rank owns one device allocation of equal size; every rank maps all of
them.  Tensors handed out by :meth:`SymmetricHeap.empty` are ordinary
``torch.Tensor`` views of the local allocation; :meth:`peer_ptr` translates a
local tensor into the address of the same object in a peer's allocation, which
the fused kernels dereference directly (P2P loads/stores over NVLink).

Back ends: ``ipc`` (cudaMalloc + CUDA IPC handles carried by the
``torch.distributed`` store) and ``vmm`` (cuMemCreate + POSIX file descriptors
passed over a Unix socket, optionally bound to an NVLS multicast object whose
mapping is :attr:`mc_base`).

The reference exchanges three cudaMalloc'ed buffers per rank with cudaIpc
(comm_comp/exp3_gemm_rs_fused.cu:368-391, comm_comp/ipc_multiproc.cuh:159-171)
and has no heap and no multicast mapping.
"""
from __future__ import annotations

import atexit
import ctypes as C
import math
import os
import socket
import time
import weakref

import torch

from .. import _native
from . import group as G


class _RawMem:
    """Exposes a raw device range through ``__cuda_array_interface__``."""

    def __init__(self, ptr: int, nbytes: int, owner=None):
        self.owner = owner
        self.__cuda_array_interface__ = {
            "shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2,
        }


def _round_up(x: int, a: int) -> int:
    return (x + a - 1) // a * a


class SymmetricHeap:
    def __init__(self, nbytes: int, backend: str = "ipc", multicast: bool = False, group=None):
        if not torch.cuda.is_available():
            raise RuntimeError("SymmetricHeap needs a CUDA device")
        self.lib = _native.lib()
        self.group = group
        self.rank = G.rank(group)
        self.world = G.world_size(group)
        self.device = torch.cuda.current_device()
        self.backend = backend
        self.mc_base: int | None = None
        self._cursor = 0
        self._opened: list[int] = []
        self._handles: list[int] = []
        torch.cuda.init()
        torch.zeros(1, device="cuda")  # make sure the primary context exists
        if backend == "ipc":
            if multicast:
                raise ValueError("multicast needs the vmm back end")
            self._init_ipc(nbytes)
        elif backend == "vmm":
            self._init_vmm(nbytes, multicast)
        else:
            raise ValueError(f"unknown heap back end {backend!r}")
        self._local = torch.as_tensor(_RawMem(self.base[self.rank], self.nbytes, self), device=f"cuda:{self.device}")
        if self.mc_base is not None:
            # A process must not end with its memory still bound to the NVLink multicast object while peers hold
            # mappings of it: whatever ends this process (an exception on another path, sys.exit), the binding is
            # taken down first, locally and without waiting for anybody.
            ref = weakref.ref(self)
            atexit.register(lambda: ref() is not None and ref().release_multicast())
        G.host_barrier(group)

    def __enter__(self):
        return self

    def __exit__(self, exc_type, exc, tb):
        if exc_type is None:
            self.close()
        else:
            # Peers may be anywhere: no collective step on the way out of a failure.
            self.release_multicast()
        return False

    def release_multicast(self) -> None:
        """Local, barrier-free teardown of the multicast binding and mapping (no-op without one, and the second
        time).  For failure paths and process exit; the orderly, collective teardown is :meth:`close`.  After
        it the heap still serves peer loads and stores, but ``mc_ptr`` addresses are gone."""
        if self.mc_base is None:
            return
        try:
            torch.cuda.synchronize()
        except Exception:  # noqa: BLE001  (a failed context must not stop the unbind)
            pass
        mc, self.mc_base = self.mc_base, None
        self.lib.tcl_mc_unbind(self._mc_handle, self.device, self.nbytes)
        self.lib.tcl_vmm_unmap(C.c_void_p(mc), self.nbytes, self._mc_handle)

    # ---- back ends -------------------------------------------------------------
    def _init_ipc(self, nbytes: int) -> None:
        self.nbytes = _round_up(nbytes, 2 << 20)
        p = C.c_void_p()
        _native.check(self.lib.tcl_heap_alloc(self.nbytes, C.byref(p)), "tcl_heap_alloc")
        torch.cuda.synchronize()
        self.base = [0] * self.world
        self.base[self.rank] = p.value
        if self.world > 1:
            hs = self.lib.tcl_ipc_handle_size()
            buf = C.create_string_buffer(hs)
            _native.check(self.lib.tcl_ipc_get_handle(p, buf), "cudaIpcGetMemHandle")
            handles = G.all_gather_object(bytes(buf.raw), self.group)
            for r, h in enumerate(handles):
                if r == self.rank:
                    continue
                q = C.c_void_p()
                _native.check(self.lib.tcl_ipc_open(C.c_char_p(h), C.byref(q)), f"cudaIpcOpenMemHandle(rank {r})")
                self.base[r] = q.value
                self._opened.append(q.value)

    def _sock_name(self, job: str, r: int) -> str:
        return f"\0tileccl-{job}-{r}"

    def _exchange_fds(self, fd: int, tag: str) -> list[int]:
        """All-to-all of one file descriptor per rank over abstract Unix sockets."""
        job = os.environ.get("TORCHELASTIC_RUN_ID", "") + os.environ.get("MASTER_PORT", "0") + tag
        srv = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
        srv.bind(self._sock_name(job, self.rank))
        srv.listen(self.world)
        G.host_barrier(self.group)
        fds = [-1] * self.world
        fds[self.rank] = fd
        # Send to every peer, then accept world-1 messages.
        for r in range(self.world):
            if r == self.rank:
                continue
            c = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
            for _ in range(200):
                try:
                    c.connect(self._sock_name(job, r))
                    break
                except OSError:
                    time.sleep(0.05)
            socket.send_fds(c, [self.rank.to_bytes(4, "little")], [fd])
            c.close()
        for _ in range(self.world - 1):
            conn, _addr = srv.accept()
            msg, got, _flags, _a = socket.recv_fds(conn, 4, 1)
            fds[int.from_bytes(msg, "little")] = got[0]
            conn.close()
        srv.close()
        G.host_barrier(self.group)
        return fds

    def _init_vmm(self, nbytes: int, multicast: bool) -> None:
        gran = C.c_size_t()
        _native.check(self.lib.tcl_vmm_granularity(self.device, C.byref(gran), 0, self.world), "granularity")
        g = gran.value
        if multicast:
            if not self.lib.tcl_multicast_supported(self.device):
                raise RuntimeError("this device does not support multicast objects")
            mg = C.c_size_t()
            _native.check(self.lib.tcl_vmm_granularity(self.device, C.byref(mg), 1, self.world), "mc granularity")
            g = g * mg.value // math.gcd(g, mg.value)
        self._gran = g
        self.nbytes = _round_up(nbytes, g)
        h, fd, p = C.c_uint64(), C.c_int(), C.c_void_p()
        _native.check(self.lib.tcl_vmm_create(self.device, self.nbytes, g, C.byref(h), C.byref(fd), C.byref(p)), "cuMemCreate")
        torch.cuda.synchronize()
        self._handles.append(h.value)
        self.base = [0] * self.world
        self.base[self.rank] = p.value
        self._local_handle = h.value
        if self.world > 1:
            fds = self._exchange_fds(fd.value, "mem")
            for r in range(self.world):
                if r == self.rank:
                    continue
                hh, q = C.c_uint64(), C.c_void_p()
                _native.check(self.lib.tcl_vmm_import(self.device, fds[r], self.nbytes, g, C.byref(hh), C.byref(q)), f"import rank {r}")
                os.close(fds[r])
                self.base[r] = q.value
                self._handles.append(hh.value)
        os.close(fd.value)
        if multicast and self.world > 1:
            mc = C.c_uint64()
            if self.rank == 0:
                mfd = C.c_int()
                _native.check(self.lib.tcl_mc_create(self.world, self.nbytes, C.byref(mc), C.byref(mfd)), "cuMulticastCreate")
                my_fd = mfd.value
            else:
                my_fd = os.open("/dev/null", os.O_RDONLY)
            fds = self._exchange_fds(my_fd, "mc")
            if self.rank != 0:
                _native.check(self.lib.tcl_mc_import(fds[0], C.byref(mc)), "import multicast")
            for r, f in enumerate(fds):
                if f >= 0:
                    os.close(f)
            _native.check(self.lib.tcl_mc_add_device(mc.value, self.device), "cuMulticastAddDevice")
            G.host_barrier(self.group)
            q = C.c_void_p()
            _native.check(self.lib.tcl_mc_bind_and_map(mc.value, self._local_handle, self.nbytes, g, self.device, C.byref(q)), "cuMulticastBindMem")
            self.mc_base = q.value
            self._mc_handle = mc.value
            G.host_barrier(self.group)

    # ---- allocation ------------------------------------------------------------
    def alloc_bytes(self, nbytes: int, align: int = 1024) -> int:
        """Bump-allocates; returns the byte offset.  Every rank must make the
        same sequence of calls so that offsets agree."""
        off = _round_up(self._cursor, align)
        if off + nbytes > self.nbytes:
            raise MemoryError(f"symmetric heap exhausted: want {nbytes} at {off}, size {self.nbytes}")
        self._cursor = off + nbytes
        return off

    def empty(self, shape, dtype=torch.bfloat16, align: int = 1024) -> torch.Tensor:
        shape = tuple(int(s) for s in (shape if isinstance(shape, (tuple, list)) else (shape,)))
        n = 1
        for s in shape:
            n *= s
        esz = torch.empty((), dtype=dtype).element_size()
        off = self.alloc_bytes(n * esz, align)
        return self._local[off: off + n * esz].view(dtype).view(shape)

    def zeros(self, shape, dtype=torch.int32, align: int = 1024) -> torch.Tensor:
        t = self.empty(shape, dtype, align)
        t.zero_()
        return t

    def offset_of(self, t: torch.Tensor) -> int:
        off = t.data_ptr() - self.base[self.rank]
        if off < 0 or off >= self.nbytes:
            raise ValueError("tensor does not live in this symmetric heap")
        return off

    def peer_ptr(self, t: torch.Tensor, r: int) -> int:
        """Address of the same object in rank ``r``'s allocation, as mapped here."""
        return self.base[r] + self.offset_of(t)

    def mc_ptr(self, t: torch.Tensor) -> int:
        if self.mc_base is None:
            raise RuntimeError("heap has no multicast mapping")
        return self.mc_base + self.offset_of(t)

    def peer_tensor(self, t: torch.Tensor, r: int) -> torch.Tensor:
        """A tensor view of rank ``r``'s copy of ``t`` (debugging / verification only)."""
        nbytes = t.numel() * t.element_size()
        raw = torch.as_tensor(_RawMem(self.peer_ptr(t, r), nbytes, self), device=f"cuda:{self.device}")
        return raw.view(t.dtype).view(t.shape)

    def reset(self) -> None:
        """Forget every allocation (the memory stays mapped)."""
        self._cursor = 0

    def close(self) -> None:
        torch.cuda.synchronize()
        G.host_barrier(self.group)
        if self.backend == "ipc":
            for p in self._opened:
                self.lib.tcl_ipc_close(C.c_void_p(p))
            self._opened = []
            G.host_barrier(self.group)
            if self.base[self.rank]:
                self.lib.tcl_heap_free(C.c_void_p(self.base[self.rank]))
                self.base[self.rank] = 0
        elif self.backend == "vmm" and self.base[self.rank]:
            # Order matters: nobody may lose its memory while a peer can still reach it through the
            # multicast object or a peer mapping.  Every step is followed by a host barrier.
            self.release_multicast()
            G.host_barrier(self.group)
            own = self._handles[0]
            for r, h in zip([x for x in range(self.world) if x != self.rank], self._handles[1:]):
                self.lib.tcl_vmm_unmap(C.c_void_p(self.base[r]), self.nbytes, h)
                self.base[r] = 0
            G.host_barrier(self.group)
            self.lib.tcl_vmm_unmap(C.c_void_p(self.base[self.rank]), self.nbytes, own)
            self.base[self.rank] = 0
            self._handles = []
