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


def zero_scale_padding(sf_swizzled: torch.Tensor, rows: int, k: int, block: int = 16) -> torch.Tensor:
    """Zeroes, in place, the padding bytes of a swizzled scale tensor [round_up(rows,128), round_up(k/block,4)]: the
    rows beyond `rows` and the scale columns beyond k/block.  For scale tensors that did not come from this
    package's quantizers (weights imported from another tool; the reference's own quantizer leaves these bytes
    uninitialised, nvfp/_ops_real.py:46-54 there).  The GEMM needs it when k is not a multiple of 4*block: the last
    MMA then covers scale columns past k/block whose operand bytes read as zero, and a non-finite scale byte there
    (0x7F / 0xFF as ue4m3, 0xFF as ue8m0) would turn 0 * scale into NaN.  Works on CPU and CUDA tensors of any
    one-byte dtype; returns the tensor."""
    rows_padded, cols_padded = sf_swizzled.shape
    if rows_padded % 128 or cols_padded % 4 or rows_padded < rows or cols_padded * block < k:
        raise ValueError(f"scale tensor {tuple(sf_swizzled.shape)} does not match a padded [{rows}, {k}] operand")
    raw = sf_swizzled.view(torch.uint8)
    # [rowTile][kTile][32][4][4] (reference: kernel/nvfp4_utils.cuh:126-153): row = 128*rt + 32*i4 + r32, col = 4*kt + c
    tiles = raw.reshape(rows_padded // 128, cols_padded // 4, 32, 4, 4)
    dev = raw.device
    row = (torch.arange(rows_padded // 128, device=dev).view(-1, 1, 1, 1, 1) * 128 +
           torch.arange(4, device=dev).view(1, 1, 1, 4, 1) * 32 + torch.arange(32, device=dev).view(1, 1, 32, 1, 1))
    col = torch.arange(cols_padded // 4, device=dev).view(1, -1, 1, 1, 1) * 4 + torch.arange(4, device=dev).view(1, 1, 1, 1, 4)
    tiles.masked_fill_((row >= rows) | (col >= k // block), 0)
    return sf_swizzled
