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
from nvfp_kernel_b200.sharding import gather_columns_layout, shard_columns, shard_range, shard_rows, zero_scale_padding
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


@pytest.mark.parametrize("rows,k,block", [(129, 80, 16), (300, 96, 16), (128, 64, 16), (17, 320, 32), (1, 32, 16)])
def test_zero_scale_padding_clears_exactly_the_padding(rows, k, block):
    """A foreign scale tensor with garbage (here: NaN patterns) in its padding: after the helper the valid region
    is untouched and every padding byte is zero, judged through the oracle's de-swizzle."""
    rp, cp = (rows + 127) // 128 * 128, (k // block + 3) // 4 * 4
    rng = np.random.default_rng(5)
    lin = rng.integers(1, 0x7E, size=(rp, cp), dtype=np.uint8)
    lin[rows:, :] = 0xFF
    lin[:, k // block:] = 0x7F
    swz = torch.from_numpy(O.swizzle_128x4(lin[:rows, :k // block]).copy())
    # the oracle's swizzle pads with zeros; put the garbage back in through the inverse view
    full = torch.from_numpy(lin).reshape(rp // 128, 4, 32, cp // 4, 4).permute(0, 3, 2, 1, 4).reshape(rp, cp).contiguous()
    assert np.array_equal(O.unswizzle_128x4(full.numpy(), rows, k // block), lin[:rows, :k // block])
    out = zero_scale_padding(full.clone(), rows, k, block)
    assert np.array_equal(out.numpy(), swz.numpy())
    with pytest.raises(ValueError):
        zero_scale_padding(torch.zeros((rp, cp + 1), dtype=torch.uint8), rows, k, block)


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


def test_gate_up_interleave_layout_and_mlp_shard_granules():
    """Rows of the fused gate/up weight come in groups of 16 gate rows followed by their 16 up rows, so that output
    columns [32g, 32g+16) and [32g+16, 32g+32) of the GEMM are gate and up of the same 16 hidden units; a rank's
    shard of the interleaved tensor is the interleave of its shards."""
    from nvfp_kernel_b200._ops_real import interleave_gate_up
    inter, k = 256, 64
    gate = torch.arange(inter * k, dtype=torch.float32).reshape(inter, k)
    up = -gate
    gu = interleave_gate_up(gate, up)
    assert gu.shape == (2 * inter, k)
    for g in range(inter // 16):
        assert torch.equal(gu[32 * g:32 * g + 16], gate[16 * g:16 * g + 16])
        assert torch.equal(gu[32 * g + 16:32 * g + 32], up[16 * g:16 * g + 16])
    world = 2
    for rank in range(world):
        lo, hi = shard_range(inter, rank, world, 64, "intermediate_size")
        assert torch.equal(gu[2 * lo:2 * hi], interleave_gate_up(gate[lo:hi], up[lo:hi]))
    with pytest.raises(AssertionError):
        interleave_gate_up(gate[:24], up[:24])
    with pytest.raises(ValueError):
        shard_range(192, 0, 2, 64, "intermediate_size")      # 96 per rank is not a multiple of 64


def test_model_surgery_leaves_models_it_cannot_run_alone():
    """quantize_gated_mlps / quantize_linear_layers on a CPU model: nothing qualifies (the kernels need CUDA weights),
    nothing is replaced and the calibration run is not started; SiLU detection by class and by name."""
    import torch.nn as nn
    from nvfp_kernel_b200.convert import _is_silu, quantize_gated_mlps, quantize_linear_layers

    class MLP(nn.Module):
        def __init__(self, act):
            super().__init__()
            self.gate_proj = nn.Linear(64, 128, bias=False)
            self.up_proj = nn.Linear(64, 128, bias=False)
            self.down_proj = nn.Linear(128, 64, bias=False)
            self.act_fn = act

    def swish(x):
        return x * torch.sigmoid(x)

    assert _is_silu(MLP(nn.SiLU())) and _is_silu(MLP(swish)) and not _is_silu(MLP(nn.GELU()))
    assert not _is_silu(nn.Linear(4, 4))
    model = nn.Sequential(MLP(nn.SiLU()))
    called = []
    assert quantize_gated_mlps(model, lambda: called.append(1)) == [] and not called
    assert quantize_linear_layers(model) == []
    assert isinstance(model[0].gate_proj, nn.Linear)
