"""Peer-visible buffers of the tensor-parallel layers' fused collectives.

Column-parallel (`GatherBuffer`): every rank owns a symmetric buffer holding the gathered [M, N] matrix; rank r's GEMM
epilogue writes its [M, N_local] slab into columns [r*N_local, (r+1)*N_local) of EVERY rank's buffer over NVLink (plain
peer stores issued by TMA, no multicast), so no collective runs afterwards.  Row-parallel (`ReduceBuffer`): every rank
owns the fp32 rows of the sum it is responsible for, and every rank's epilogue adds its partial product's rows into
their owner's buffer.

The ranks are synchronised inside the GEMM kernel through a block of flag words that lives beside each buffer
(include/nvfp_b200.h, nvfp_peer_group_t): no barrier kernel and no collective surrounds the call, and every wait on a
peer is bounded.  torch.distributed._symmetric_memory is plumbing here: allocation and address exchange.
"""
from __future__ import annotations

import os

import torch

FLAG_WORDS = 32          # NVFP_PEER_FLAG_WORDS


class _PeerBuffer:
    def __init__(self, shape, dtype: torch.dtype, device, group=None):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem

        # plain peer mappings only: do not bind the buffers to an NVLink multicast object
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.buf = symm_mem.empty(shape, dtype=dtype, device=device)
        self.flags = symm_mem.empty((FLAG_WORDS,), dtype=torch.int32, device=device)
        self.flags.zero_()
        self.handle = symm_mem.rendezvous(self.buf, group)
        self.flag_handle = symm_mem.rendezvous(self.flags, group)
        self.buffer_ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.flag_ptrs = [int(p) for p in self.flag_handle.buffer_ptrs]       # rank order
        # every rank's flag block is zero before anybody announces anything in it (once, at construction)
        torch.cuda.synchronize(device)
        dist.barrier(group)
        # bound of each in-kernel wait on a peer, nanoseconds; 0 = the library's default (two seconds)
        self.wait_limit_ns = 0


class GatherBuffer(_PeerBuffer):
    def __init__(self, m: int, n_local: int, dtype: torch.dtype, device, group=None):
        import torch.distributed as dist
        world = dist.get_world_size(group if group is not None else dist.group.WORLD)
        super().__init__((m, world * n_local), dtype, device, group)
        self.m, self.n_local, self.dtype = m, n_local, dtype
        self.ld = self.world * n_local
        col_offset = self.rank * n_local * self.buf.element_size()
        # rank r's entry: where THIS rank's slab starts in rank r's gathered matrix
        self.dst_ptrs = [p + col_offset for p in self.buffer_ptrs]

    def gathered(self) -> torch.Tensor:
        """The local [M, N] buffer."""
        return self.buf


class ReduceBuffer(_PeerBuffer):
    """fp32 [M / world, N] accumulation buffer of the row-parallel layer's fused reduce-scatter: every
    rank's GEMM epilogue adds its partial product's rows into the buffer of the rank that owns them."""

    def __init__(self, m: int, n: int, device, group=None):
        import torch.distributed as dist
        world = dist.get_world_size(group if group is not None else dist.group.WORLD)
        assert m % (32 * world) == 0, "fused reduce-scatter needs M to be a multiple of 32 x world size"
        super().__init__((m // world, n), torch.float32, device, group)
        self.dst_ptrs = self.buffer_ptrs                                  # destination r = rank r's buffer


class Fp4GatherBuffer(_PeerBuffer):
    """Gathered NVFP4 operand of a column-parallel layer: packed nibbles [M, N / 2] and swizzled scale bytes
    [round_up(M, 128), N / 16] of the whole [M, N] matrix, in one peer-visible allocation per rank.  Every rank's GEMM
    epilogue quantizes its tiles and stores bytes and scales of its N_local columns into every rank's buffer."""

    def __init__(self, m: int, n_local: int, device, group=None):
        import torch.distributed as dist
        world = dist.get_world_size(group if group is not None else dist.group.WORLD)
        n = world * n_local
        assert n_local % 64 == 0, "the NVFP4 gather needs whole 64-column scale chunks per rank"
        self.m, self.n, self.n_local = m, n, n_local
        rows_padded = (m + 127) // 128 * 128
        self.packed_bytes = (m * (n // 2) + 255) // 256 * 256
        self.sf_bytes = rows_padded * (n // 16)
        super().__init__((self.packed_bytes + self.sf_bytes,), torch.uint8, device, group)
        self.packed = self.buf[:m * (n // 2)].view(m, n // 2)
        self.scales = self.buf[self.packed_bytes:].view(rows_padded, n // 16)
        self.packed_ptrs = self.buffer_ptrs
        self.sf_ptrs = [p + self.packed_bytes for p in self.buffer_ptrs]
        self.n_offset = self.rank * n_local
