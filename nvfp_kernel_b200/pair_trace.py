"""Where the CTA-pair GEMM's roles wait: runs the instrumented build of the library.

    python -m nvfp_kernel_b200.build --trace
    python -m nvfp_kernel_b200.pair_trace [M N K]          # default 8192 8192 8192

libnvfp_b200_trace.so is libnvfp_b200.so compiled with -DNVFP_PAIR_TRACE: the one thread that issues the MMAs of a CTA
pair, the leader's producer thread and the leader's first epilogue warp add up the clocks they spend in each of their
waits (clock64 around the wait, nothing else changes).  The kernel is timed with CUDA events like any other, the
counters are read afterwards; clocks are per cluster, the table gives mean and range over the clusters.
"""
from __future__ import annotations

import ctypes
import os
import sys

import torch

from . import _capi, ops

TRACE_LIB = os.path.join(os.path.dirname(os.path.abspath(__file__)), "libnvfp_b200_trace.so")
COLUMNS = ("issuer total", "issuer: operands not there", "issuer: accumulator busy", "K stages", "producer: no free stage",
           "epilogue: tile not finished", "epilogue: staging not drained", "tiles")


def main():
    m, n, k = (int(v) for v in sys.argv[1:4]) if len(sys.argv) >= 4 else (8192, 8192, 8192)
    if not os.path.exists(TRACE_LIB):
        raise SystemExit(f"{TRACE_LIB} is missing: python -m nvfp_kernel_b200.build --trace")
    lib = ctypes.CDLL(TRACE_LIB)
    lib.nvfp_scaled_fp4_mm.restype = ctypes.c_int
    lib.nvfp_scaled_fp4_mm.argtypes = _capi.PROTOTYPES["nvfp_scaled_fp4_mm"][1]
    lib.nvfp_debug_pair_trace.restype = ctypes.c_int
    lib.nvfp_debug_pair_trace.argtypes = [ctypes.c_void_p, ctypes.c_int]
    a = torch.randn(m, k, device="cuda").to(torch.bfloat16)
    w = torch.randn(n, k, device="cuda").to(torch.bfloat16)
    ga, gw = ops.global_scale(a), ops.global_scale(w)
    a4, asf = ops.scaled_fp4_quant(a, ga)
    w4, wsf = ops.scaled_fp4_quant(w, gw)
    alpha = ops.alpha_from_scales(ga, gw)
    out = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    args = (out.data_ptr(), a4.data_ptr(), w4.data_ptr(), asf.data_ptr(), wsf.data_ptr(), alpha.data_ptr(), m, n, k,
            _capi.NVFP_DTYPE_BF16, stream)
    clusters = min(74, ((m + 255) // 256) * ((n + 255) // 256))
    buf = (ctypes.c_uint64 * (8 * clusters))()
    for _ in range(3):
        assert lib.nvfp_scaled_fp4_mm(*args) == 0
    assert lib.nvfp_debug_pair_trace(buf, clusters) == 0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    assert lib.nvfp_scaled_fp4_mm(*args) == 0
    e1.record()
    torch.cuda.synchronize()
    assert lib.nvfp_debug_pair_trace(buf, clusters) == 0
    t = torch.tensor(list(buf), dtype=torch.float64).view(clusters, 8)
    print(f"fp4_gemm_pair_kernel (instrumented) {m} x {n} x {k}: {e0.elapsed_time(e1) * 1e3:.1f} us, {clusters} clusters")
    total = t[:, 0].mean().item()
    print(f"{'':34s} {'mean clk':>12s} {'min':>12s} {'max':>12s} {'share of issuer total':>22s}")
    for i, name in enumerate(COLUMNS):
        col = t[:, i]
        share = f"{col.mean().item() / total:22.1%}" if i not in (0, 3, 7) else f"{'':22s}"
        print(f"{name:34s} {col.mean().item():12.0f} {col.min().item():12.0f} {col.max().item():12.0f} {share}")
    stages = t[:, 3].mean().item()
    print(f"issuer clocks per K stage of 256: {total / stages:.0f} (4 MMAs of 128 clk = 512 when the tensor pipe never waits)")


if __name__ == "__main__":
    main()
