"""Tensor-parallel QuantLinear on 2 GPUs of one box (skipped with fewer): column-parallel with the
NCCL all-gather and with the gather fused into the GEMM epilogue (peer stores) must both equal the
1-GPU result bit for bit; row-parallel (K-split, reduce-scatter) stays within the GEMM tolerance; the
tensor-parallel gated MLP (fused activation and quantization, NCCL or fused reduce-scatter) matches the 1-GPU one."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from helpers import check_gemm
from inputs import gemm_inputs

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0",
                      TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from nvfp_kernel_b200 import QuantLinear
        m, n, k = 512, 1024, 1024
        a, w = gemm_inputs(m, n, k, seed=7, w_std=0.05)
        a, w = a.cuda(), w.cuda()
        single = QuantLinear(k, n, device="cuda").load_weight(w)(a)
        col = QuantLinear(k, n, parallel="column", device="cuda").load_weight(w)
        y_nccl = col(a)
        fused = QuantLinear(k, n, parallel="column", fused_gather=True, device="cuda").load_weight(w)
        y_fused = fused(a).clone()
        y_fused2 = fused(a * 0.5).clone()          # second call reuses the peer-visible buffer
        single2 = QuantLinear(k, n, device="cuda").load_weight(w)(a * 0.5)
        row = QuantLinear(k, n, parallel="row", device="cuda").load_weight(w)
        y_row = row(a)                                # [m / world, n]: this rank's rows
        lo, hi = rank * m // world, (rank + 1) * m // world
        check_gemm(y_row, single[lo:hi].double(), rel=2e-2)
        row_fused = QuantLinear(k, n, parallel="row", fused_reduce_scatter=True, device="cuda").load_weight(w)
        for scale in (1.0, 0.25):                   # two calls: the accumulation buffer is reused
            y_rf = row_fused(a * scale)
            ref = QuantLinear(k, n, device="cuda").load_weight(w)(a * scale)
            check_gemm(y_rf, ref[lo:hi].double(), rel=2e-2)
        # A peer that is late: rank 1 reaches the call half a second after rank 0, whose in-kernel waits are limited
        # to 20 ms.  Rank 0's kernel gives up on rank 1 (status bit 0x20), skips its stores to it and returns; rank 1
        # finds rank 0's announcements already there and completes normally.  Nothing hangs, the context stays
        # usable, and the next call (default limit again) is bit-exact on both ranks.
        import time
        import nvfp_kernel_b200 as nv
        torch.cuda.synchronize()
        assert nv.device_status() == 0
        dist.barrier()
        fused.peer_wait_limit_ns = 20_000_000
        if rank == 1:
            time.sleep(0.5)
        t0 = time.perf_counter()
        fused(a)
        torch.cuda.synchronize()
        waited = time.perf_counter() - t0
        late_status = nv.device_status()
        dist.barrier()
        fused.peer_wait_limit_ns = 0
        y_after = fused(a).clone()
        torch.cuda.synchronize()
        late_ok = (late_status == (0x20 if rank == 0 else 0)) and waited < 0.4 and bool(torch.equal(y_after, single)) \
            and nv.device_status() == 0
        # gather of the NVFP4 form of the output: the gathered operand equals the quantizer's bytes on the 1-GPU result
        out_gs = (2688.0 / single.abs().max().float()).reshape(1)
        want_fp4, want_sf = nv.scaled_fp4_quant(single, out_gs)
        fp4_ok = True
        for _ in range(2):
            g_fp4, g_sf = fused.forward_gather_fp4(a, out_gs)
            fp4_ok = fp4_ok and bool(torch.equal(g_fp4, want_fp4)) and bool(torch.equal(g_sf.view(torch.uint8), want_sf.view(torch.uint8)))
        late_ok = late_ok and fp4_ok
        # MXFP4 row-parallel: fp32 partial products through NCCL, and through the fused reduce-scatter
        single_mx = QuantLinear(k, n, format="mxfp4", device="cuda").load_weight(w)(a)
        for fused_rs in (False, True):
            row_mx = QuantLinear(k, n, format="mxfp4", parallel="row", fused_reduce_scatter=fused_rs, device="cuda").load_weight(w)
            for _ in range(2):
                check_gemm(row_mx(a), single_mx[lo:hi].double(), rel=2e-2)
        # tensor-parallel gated MLP: intermediate dimension split, hidden activation quantized in the gate/up epilogue
        # with one calibrated scale on every rank, partial sums of the down projection reduce-scattered over the rows
        from nvfp_kernel_b200 import QuantGatedMLP
        hidden, inter = 512, 1024
        g = torch.Generator().manual_seed(3)
        wg = (torch.randn(inter, hidden, generator=g) * 0.05).to(torch.bfloat16).cuda()
        wu = (torch.randn(inter, hidden, generator=g) * 0.05).to(torch.bfloat16).cuda()
        wd = (torch.randn(hidden, inter, generator=g) * 0.03).to(torch.bfloat16).cuda()
        xm = torch.randn(m, hidden, generator=g).to(torch.bfloat16).cuda()
        one = QuantGatedMLP(hidden, inter, device="cuda").load_weights(wg, wu, wd).calibrate(xm)
        y_one = one(xm)
        mlp_ok = []
        for fused_rs in (False, True):
            tp = QuantGatedMLP(hidden, inter, parallel="tensor", fused_reduce_scatter=fused_rs, device="cuda")
            tp.load_weights(wg, wu, wd).calibrate(xm)
            mlp_ok.append(bool(torch.equal(tp.act_global_scale, one.act_global_scale)))
            for scale in (1.0, 0.5):
                y_tp = tp(xm * scale)
                check_gemm(y_tp, one(xm * scale)[lo:hi].double(), rel=2e-2)
        torch.cuda.synchronize()
        ret[rank] = (bool(torch.equal(y_nccl, single)), bool(torch.equal(y_fused, single)),
                     bool(torch.equal(y_fused2, single2)), tuple(y_row.shape), tuple(mlp_ok), tuple(y_one.shape),
                     late_ok or (late_status, waited))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_column_and_row_parallel_two_gpus():
    world = 2
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    for rank in range(world):
        assert ret[rank] == (True, True, True, (256, 1024), (True, True), (512, 512), True), (rank, ret[rank])
