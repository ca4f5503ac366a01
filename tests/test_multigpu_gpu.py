"""Tensor-parallel QuantLinear on 2 GPUs of one box (skipped with fewer): column-parallel with the
NCCL all-gather and with the gather fused into the GEMM epilogue (peer stores) must both equal the
1-GPU result bit for bit; row-parallel (K-split, reduce-scatter) stays within the GEMM tolerance."""
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
        torch.cuda.synchronize()
        ret[rank] = (bool(torch.equal(y_nccl, single)), bool(torch.equal(y_fused, single)),
                     bool(torch.equal(y_fused2, single2)), tuple(y_row.shape))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_column_and_row_parallel_two_gpus():
    world = 2
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    for rank in range(world):
        assert ret[rank] == (True, True, True, (256, 1024)), (rank, ret[rank])
