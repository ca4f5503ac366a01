"""Host-side sharding of quantized operands for tensor-parallel QuantLinear layers.

Pure tensor slicing, usable on CPU tensors (the multi-process tests run it under gloo).
The reference has no distributed code; the partitions follow the two natural shardings
of a linear layer  y = x @ W^T  with W [N, K]:

  column-parallel  W split on N.  Weights are quantized BEFORE sharding with the
                   full-tensor global scale, so a shard is a slice of the 1-GPU tensors.
                   A 128-row scale tile must not straddle ranks: (N / world) % 128 == 0.
  row-parallel     W (and x) split on K.  A 512-byte scale chunk covers 4 scale columns
                   (64 elements of K for NVFP4, 128 for MXFP4); shards keep whole chunks:
                   (K / world) % (4 * block) == 0.
"""
from __future__ import annotations

import torch


def shard_range(total: int, rank: int, world: int, granule: int, what: str) -> tuple[int, int]:
    if total % world != 0 or (total // world) % granule != 0:
        raise ValueError(f"{what}={total} cannot be split over {world} ranks in multiples of {granule}")
    per = total // world
    return rank * per, (rank + 1) * per


def shard_columns(w_fp4: torch.Tensor, w_sf: torch.Tensor, rank: int, world: int):
    """N-split of packed weights [N, K/2] and swizzled scales [round_up(N,128), sf_cols]."""
    n = w_fp4.shape[0]
    lo, hi = shard_range(n, rank, world, 128, "out_features")
    return w_fp4[lo:hi].contiguous(), w_sf[lo:hi].contiguous()


def shard_rows(w_fp4: torch.Tensor, w_sf: torch.Tensor, rank: int, world: int, block: int = 16):
    """K-split of packed weights [N, K/2] and swizzled scales."""
    n, kh = w_fp4.shape
    k = kh * 2
    lo, hi = shard_range(k, rank, world, 4 * block, "in_features")
    rows_padded, sf_cols = w_sf.shape
    if sf_cols * block != k:
        raise ValueError("scale tensor does not match the weight's K (K must be a multiple of 4*block)")
    chunks = sf_cols // 4
    sf3 = w_sf.reshape(rows_padded // 128, chunks, 512)
    c_lo, c_hi = lo // (4 * block), hi // (4 * block)
    sf_shard = sf3[:, c_lo:c_hi, :].contiguous().reshape(rows_padded, (c_hi - c_lo) * 4)
    return w_fp4[:, lo // 2: hi // 2].contiguous(), sf_shard


def gather_columns_layout(parts: torch.Tensor) -> torch.Tensor:
    """[world, M, N/world] (the layout all_gather_into_tensor produces) -> [M, N]."""
    world, m, n_local = parts.shape
    return parts.permute(1, 0, 2).reshape(m, world * n_local)
