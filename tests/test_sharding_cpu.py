"""Host-side logic of the tensor-parallel layers: shard slicing of quantized operands
(single process) and the collective plumbing with world_size 2 over gloo."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from inputs import make_input
from nvfp_kernel_b200.sharding import gather_columns_layout, shard_columns, shard_range, shard_rows
from oracle import nvfp_oracle as O


def _quantized(n, k, block=16, seed=0):
    w = make_input("normal", (n, k), torch.bfloat16, seed)
    gs = O.global_scale_from_amax(w.float().abs().max().item())
    if block == 16:
        fp4, sf, _ = O.nvfp4_quantize_kernel(w, gs)
    else:
        fp4, sf, _ = O.mxfp4_quantize(w)
    return w, gs, torch.from_numpy(fp4), torch.from_numpy(sf)


def test_shard_range_rejects_ragged_splits():
    assert shard_range(512, 1, 2, 128, "n") == (256, 512)
    with pytest.raises(ValueError):
        shard_range(384, 0, 2, 128, "n")
    with pytest.raises(ValueError):
        shard_range(500, 0, 2, 4, "n")


def test_column_shards_are_slices_of_the_full_quantization():
    w, gs, fp4, sf = _quantized(512, 128)
    for rank in range(2):
        s_fp4, s_sf = shard_columns(fp4, sf, rank, 2)
        # quantizing the slice with the FULL tensor's global scale gives the same bytes
        e_fp4, e_sf, _ = O.nvfp4_quantize_kernel(w[rank * 256:(rank + 1) * 256], gs)
        assert np.array_equal(s_fp4.numpy(), e_fp4) and np.array_equal(s_sf.numpy(), e_sf)


@pytest.mark.parametrize("block", [16, 32])
def test_row_shards_are_slices_of_the_full_quantization(block):
    w, gs, fp4, sf = _quantized(256, 512, block)
    for rank in range(2):
        s_fp4, s_sf = shard_rows(fp4, sf, rank, 2, block)
        sl = w[:, rank * 256:(rank + 1) * 256].contiguous()
        if block == 16:
            e_fp4, e_sf, _ = O.nvfp4_quantize_kernel(sl, gs)
        else:
            e_fp4, e_sf, _ = O.mxfp4_quantize(sl)
        assert np.array_equal(s_fp4.numpy(), e_fp4) and np.array_equal(s_sf.numpy(), e_sf)
    # partial products of the shards add up to the full product
    a = make_input("normal", (32, 512), torch.bfloat16, 3)
    ga = O.global_scale_from_amax(a.float().abs().max().item())
    if block == 16:
        af, asf, _ = O.nvfp4_quantize_kernel(a, ga)
        kw = dict(block=16, scale_format="e4m3")
    else:
        af, asf, _ = O.mxfp4_quantize(a)
        kw = dict(block=32, scale_format="e8m0")
    full = O.scaled_mm_reference(af, fp4.numpy(), asf, sf.numpy(), 1.0, **kw)
    parts = 0
    for rank in range(2):
        wf, wsf = shard_rows(fp4, sf, rank, 2, block)
        xf, xsf = shard_rows(torch.from_numpy(af), torch.from_numpy(asf), rank, 2, block)
        parts = parts + O.scaled_mm_reference(xf.numpy(), wf.numpy(), xsf.numpy(), wsf.numpy(), 1.0, **kw)
    np.testing.assert_allclose(parts, full, rtol=1e-12, atol=1e-12)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # column-parallel: every rank computes its slab with the oracle, all-gather, re-layout
        w, gs, fp4, sf = _quantized(512, 128)
        a = make_input("normal", (16, 128), torch.bfloat16, 3)
        ga = O.global_scale_from_amax(a.float().abs().max().item())
        af, asf, _ = O.nvfp4_quantize_kernel(a, ga)
        s_fp4, s_sf = shard_columns(fp4, sf, rank, world)
        y_local = torch.from_numpy(O.scaled_mm_reference(af, s_fp4.numpy(), asf, s_sf.numpy(), 1.0))
        parts = torch.empty((world * y_local.shape[0], y_local.shape[1]), dtype=y_local.dtype)
        dist.all_gather_into_tensor(parts, y_local)
        y = gather_columns_layout(parts.view(world, *y_local.shape))
        full = torch.from_numpy(O.scaled_mm_reference(af, fp4.numpy(), asf, sf.numpy(), 1.0))
        ok_col = torch.equal(y, full)

        # row-parallel: global activation scale from a MAX all-reduce of amax bit patterns,
        # fp32 partial sums, reduce-scatter over rows
        k_lo, k_hi = shard_range(128, rank, world, 64, "k")
        a_local = a[:, k_lo:k_hi].contiguous()
        bits = a_local.float().abs().max().reshape(1).view(torch.int32).clone()
        dist.all_reduce(bits, op=dist.ReduceOp.MAX)
        ok_amax = bits.view(torch.float32).item() == a.float().abs().max().item()
        r_fp4, r_sf = shard_rows(fp4, sf, rank, world, 16)
        xf, xsf, _ = O.nvfp4_quantize_kernel(a_local, ga)
        part = torch.from_numpy(O.scaled_mm_reference(xf, r_fp4.numpy(), xsf, r_sf.numpy(), 1.0)).float()
        out = torch.empty((16 // world, 512), dtype=torch.float32)
        # gloo has no reduce_scatter_tensor: all_reduce then keep this rank's rows
        dist.all_reduce(part)
        out.copy_(part[rank * (16 // world):(rank + 1) * (16 // world)])
        ok_row = torch.allclose(out.double(), full[rank * (16 // world):(rank + 1) * (16 // world)], rtol=1e-5, atol=1e-5)
        ret[rank] = (ok_col, ok_amax, ok_row)
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_column_and_row_parallel():
    world = 2
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    assert len(ret) == world
    for rank in range(world):
        assert ret[rank] == (True, True, True), (rank, ret[rank])
