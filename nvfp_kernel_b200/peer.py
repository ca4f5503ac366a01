"""Peer-visible output buffers for the column-parallel layer's fused gather.

Every rank owns a symmetric buffer holding the gathered [M, N] matrix; rank r's GEMM epilogue writes
its [M, N_local] slab into columns [r*N_local, (r+1)*N_local) of EVERY rank's buffer over NVLink (plain peer stores issued by TMA, no multicast), so no collective runs afterwards.
Built on torch.distributed._symmetric_memory, which is plumbing here: allocation, address
exchange and a stream-ordered barrier.
"""
from __future__ import annotations

import os

import torch


class GatherBuffer:
    def __init__(self, m: int, n_local: int, dtype: torch.dtype, device, group=None):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem

        # plain peer mappings only: do not bind the buffer to an NVLink multicast object
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.m, self.n_local, self.dtype = m, n_local, dtype
        self.ld = self.world * n_local
        self.buf = symm_mem.empty((m, self.ld), dtype=dtype, device=device)
        self.handle = symm_mem.rendezvous(self.buf, group)
        col_offset = self.rank * n_local * self.buf.element_size()
        ptrs = list(self.handle.buffer_ptrs)
        # destination list for the GEMM: own buffer first, then the peers starting with the next rank, so that at
        # any moment the ranks (which walk their lists in step) write to different peers instead of all to one;
        # always this rank's columns
        order = [(self.rank + i) % self.world for i in range(self.world)]
        self.dst_ptrs = [int(ptrs[r]) + col_offset for r in order]

    def barrier(self) -> None:
        """Stream-ordered barrier over the ranks (no host synchronisation)."""
        self.handle.barrier(channel=0)

    def gathered(self) -> torch.Tensor:
        """The local [M, N] buffer."""
        return self.buf


class ReduceBuffer:
    """fp32 [M / world, N] accumulation buffer of the row-parallel layer's fused reduce-scatter: every
    rank's GEMM epilogue adds its partial product's rows into the buffer of the rank that owns them."""

    def __init__(self, m: int, n: int, device, group=None):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem

        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        assert m % (32 * self.world) == 0, "fused reduce-scatter needs M to be a multiple of 32 x world size"
        self.buf = symm_mem.empty((m // self.world, n), dtype=torch.float32, device=device)
        self.handle = symm_mem.rendezvous(self.buf, group)
        self.dst_ptrs = [int(p) for p in self.handle.buffer_ptrs]     # destination r = rank r's buffer

    def barrier(self) -> None:
        self.handle.barrier(channel=0)
