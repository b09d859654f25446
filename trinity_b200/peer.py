"""The row-parallel projection of a tensor-parallel block with its all-reduce done by the kernels over peer memory
(``tb200_gemm_peer_reduce``): one process per GPU, every rank's staging / result / flag buffers mapped into every other
rank's address space through CUDA IPC, handles exchanged once through ``torch.distributed``.

    comm = PeerReduce(m, n, torch.bfloat16, device)        # collective: every rank of the group makes the call
    out = comm.gemm_reduce(a_local, b_local)                # = sum over ranks of a_r @ b_r, complete on every rank

The reference has no multi-GPU path; this stands where ``gemm`` + ``dist.all_reduce`` would.  A communicator serves one
shape ``(m, n)``; ``out`` is the communicator's own buffer and is overwritten by the next call.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch
import torch.distributed as dist

from . import _lib as L
from . import ops


def _align(x: int, a: int = 256) -> int:
    return (x + a - 1) // a * a


class PeerReduce:
    def __init__(self, m: int, n: int, dtype: torch.dtype, device: torch.device, group=None):
        lib = L.load()
        self.lib = lib
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        if self.world > 8:
            raise ValueError("PeerReduce serves at most 8 ranks (one NVSwitch domain)")
        if m % (128 * self.world) != 0 or n % 8 != 0:
            raise ValueError(f"m must be a multiple of 128 * world = {128 * self.world} and n of 8")
        if dtype not in (torch.bfloat16, torch.float16):
            raise TypeError("PeerReduce moves 16-bit partial products")
        self.m, self.n, self.dtype, self.device, self.group = m, n, dtype, device, group
        stage_bytes = _align(int(lib.tb200_peer_stage_bytes(m, n)))
        out_bytes = _align(m * n * 2)
        sync_bytes = _align(int(lib.tb200_peer_sync_bytes(m, self.world)))
        # ONE allocation per rank (stage | out | sync): one IPC handle per peer to open
        self.block = torch.zeros(stage_bytes + out_bytes + sync_bytes, dtype=torch.uint8, device=device)
        self._off = (0, stage_bytes, stage_bytes + out_bytes)
        self.out = self.block[stage_bytes:stage_bytes + m * n * 2].view(dtype).view(m, n)
        torch.cuda.synchronize(device)
        self._opened = []
        bases = [None] * self.world
        bases[self.rank] = self.block.data_ptr()
        if self.world > 1:
            handle = (C.c_ubyte * 64)()
            offset = C.c_int64(0)
            L.check(lib.tb200_ipc_export(self.block.data_ptr(), handle, C.byref(offset)), "tb200_ipc_export")
            mine = (bytes(handle), int(offset.value))
            everyone = [None] * self.world
            dist.all_gather_object(everyone, mine, group=group)
            for r, (h, off) in enumerate(everyone):
                if r == self.rank:
                    continue
                buf = (C.c_ubyte * 64).from_buffer_copy(h)
                ptr = C.c_void_p()
                L.check(lib.tb200_ipc_open(buf, off, C.byref(ptr)), f"tb200_ipc_open (rank {r}'s buffers)")
                bases[r] = ptr.value
                self._opened.append((ptr.value, off))
            dist.barrier(group=group)          # nobody starts before everybody has mapped everybody
        self._bases = bases
        self.epoch = 0

    def _table(self, which: int):
        t = (C.c_void_p * 8)()
        for r in range(self.world):
            t[r] = self._bases[r] + self._off[which]
        return t

    def gemm_reduce(self, a: torch.Tensor, b: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``sum_r a_r @ b_r [+ residual]`` on every rank.  ``a``: (m, k_local), ``b``: (k_local, n); ``residual``: (m, n),
        the same on all ranks.  Launches on the current stream; returns the communicator's result buffer."""
        if a.shape[0] != self.m or b.shape[1] != self.n or a.shape[1] != b.shape[0] or a.dtype != self.dtype or b.dtype != self.dtype:
            raise ValueError("this communicator was set up for another shape or dtype")
        if residual is not None and (tuple(residual.shape) != (self.m, self.n) or residual.dtype != self.dtype):
            raise ValueError("residual must be (m, n) of the communicator's dtype")
        self.epoch += 1
        args = L.PeerGemmArgs(dtype=ops._dt(a), world=self.world, rank=self.rank, m=self.m, n=self.n, k=a.shape[1],
                              a=ops._ptr(a), b=ops._ptr(b), residual=ops._ptr(residual), stage=self._table(0), out=self._table(1),
                              sync=self._table(2), epoch=self.epoch)
        L.check(self.lib.tb200_gemm_peer_reduce(C.byref(args), ops._stream()), "tb200_gemm_peer_reduce")
        return self.out

    def close(self) -> None:
        """Unmap the peers' buffers (after a device synchronisation and a barrier: nobody may still be writing them)."""
        torch.cuda.synchronize(self.device)
        if self.world > 1:
            dist.barrier(group=self.group)
        for ptr, off in self._opened:
            self.lib.tb200_ipc_close(ptr, off)
        self._opened = []
