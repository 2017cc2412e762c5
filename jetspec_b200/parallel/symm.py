"""Peer-visible ("symmetric") device buffers.

Each rank allocates the same-sized buffer with the kernel library's allocator, the CUDA
IPC handles travel through the host process group, and every rank maps all peers'
buffers.  ``ptrs_dev`` is a device array of ``world`` addresses (this rank's own buffer at
index ``rank``) that the fused compute+collective kernels index by rank; they reach peer
memory with plain loads and stores over NVLink.  (No counterpart in the reference, whose only collectives are the
benchmark's NCCL reductions, ``bench/engine/tps_walltime.py:111-139``.)
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch


class SymmetricBuffer:
    def __init__(self, nbytes: int, group=None):
        import torch.distributed as dist
        from ..ops import cuda_ext as X
        lib = X.load()
        lib.js_symm_alloc.restype = ctypes.c_void_p
        lib.js_symm_alloc.argtypes = [ctypes.c_size_t]
        lib.js_symm_import.restype = ctypes.c_void_p
        lib.js_symm_export.argtypes = [ctypes.c_void_p, ctypes.c_char_p]
        lib.js_symm_free.argtypes = [ctypes.c_void_p]
        lib.js_symm_unmap.argtypes = [ctypes.c_void_p]
        self._lib = lib
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.nbytes = int(nbytes)
        self.local = lib.js_symm_alloc(self.nbytes)
        if not self.local:
            raise RuntimeError(f"symmetric allocation of {nbytes} bytes failed")
        handle = ctypes.create_string_buffer(64)
        if lib.js_symm_export(ctypes.c_void_p(self.local), handle) != 0:
            raise RuntimeError("cudaIpcGetMemHandle failed")
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(handle.raw), group=group)
        self.ptrs = []
        for r, h in enumerate(handles):
            if r == self.rank:
                self.ptrs.append(self.local)
            else:
                p = lib.js_symm_import(ctypes.c_char_p(h))
                if not p:
                    raise RuntimeError(f"mapping rank {r}'s buffer failed (cudaIpcOpenMemHandle)")
                self.ptrs.append(p)
        self.ptrs_dev = torch.tensor(self.ptrs, dtype=torch.int64, device="cuda")
        dist.barrier(group=group)

    def tensor(self, rank: int, shape, dtype, offset_bytes: int = 0) -> torch.Tensor:
        """A tensor aliasing rank ``rank``'s buffer (peer memory when ``rank`` is not this rank).  Such a
        tensor may be handed to THIS library's kernels as a destination or source; it must never be
        given to a library kernel (GEMM, attention, NCCL) as an operand."""
        typestr = {torch.bfloat16: "<u2", torch.float16: "<f2", torch.float32: "<f4", torch.int32: "<i4",
                   torch.int64: "<i8", torch.uint8: "|u1"}[dtype]

        class _Alias:
            pass
        a = _Alias()
        a.__cuda_array_interface__ = {"shape": tuple(int(s) for s in shape), "typestr": typestr,
                                      "data": (int(self.ptrs[rank]) + int(offset_bytes), False), "version": 3}
        t = torch.as_tensor(a, device="cuda")
        return t.view(torch.bfloat16) if dtype == torch.bfloat16 else t

    def zero_local(self) -> None:
        self.tensor(self.rank, (self.nbytes,), torch.uint8).zero_()

    def close(self) -> None:
        for r, p in enumerate(self.ptrs):
            if r != self.rank and p:
                self._lib.js_symm_unmap(ctypes.c_void_p(p))
        if self.local:
            self._lib.js_symm_free(ctypes.c_void_p(self.local))
        self.ptrs, self.local = [], None
