"""Where the CTA-pair GEMM's roles wait: runs the instrumented build of the library.

    python -m nvfp_kernel_b200.build --trace
    python -m nvfp_kernel_b200.pair_trace [M N K [PAIRS [noloads]]]  # default 8192 8192 8192, every CTA pair of the GPU

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
SLOTS = 16
COLUMNS = ("issuer total", "issuer: operands not there", "issuer: accumulator busy", "K stages", "producer: no free stage",
           "epilogue: tile not finished", "epilogue: staging not drained", "tiles")


def main():
    m, n, k = (int(v) for v in sys.argv[1:4]) if len(sys.argv) >= 4 else (8192, 8192, 8192)
    max_pairs = int(sys.argv[4]) if len(sys.argv) >= 5 else 74
    no_loads = len(sys.argv) >= 6 and sys.argv[5] == "noloads"
    os.environ["NVFP_TRACE_MAX_PAIRS"] = str(max_pairs)      # read by the instrumented library at each launch
    os.environ["NVFP_TRACE_NO_LOADS"] = "1" if no_loads else "0"
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
    clusters = min(74, max_pairs, ((m + 255) // 256) * ((n + 255) // 256))
    buf = (ctypes.c_uint64 * (SLOTS * clusters))()
    for _ in range(3):
        assert lib.nvfp_scaled_fp4_mm(*args) == 0
    assert lib.nvfp_debug_pair_trace(buf, clusters) == 0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    assert lib.nvfp_scaled_fp4_mm(*args) == 0
    e1.record()
    torch.cuda.synchronize()
    assert lib.nvfp_debug_pair_trace(buf, clusters) == 0
    t = torch.tensor(list(buf), dtype=torch.float64).view(clusters, SLOTS)
    print(f"fp4_gemm_pair_kernel (instrumented) {m} x {n} x {k}: {e0.elapsed_time(e1) * 1e3:.1f} us, {clusters} clusters")
    total = t[:, 0].mean().item()
    print(f"{'':34s} {'mean clk':>12s} {'min':>12s} {'max':>12s} {'share of issuer total':>22s}")
    for i, name in enumerate(COLUMNS):
        col = t[:, i]
        share = f"{col.mean().item() / total:22.1%}" if i not in (0, 3, 7) else f"{'':22s}"
        print(f"{name:34s} {col.mean().item():12.0f} {col.min().item():12.0f} {col.max().item():12.0f} {share}")
    # slots 8..10 are sums of clock values over the tiles that have a successor: keep them as integers
    raw = [int(v) for v in buf]
    seen = sum(raw[c * SLOTS + 9] for c in range(clusters))
    released = sum(raw[c * SLOTS + 10] for c in range(clusters))
    taken = sum(raw[c * SLOTS + 8] for c in range(clusters))
    loaded = sum(raw[c * SLOTS + 11] for c in range(clusters))
    ld_issued = sum(raw[c * SLOTS + 12] for c in range(clusters))
    fenced = sum(raw[c * SLOTS + 13] for c in range(clusters))
    first_ld = sum(raw[c * SLOTS + 14] for c in range(clusters))
    handovers = sum(raw[c * SLOTS + 7] - 1 for c in range(clusters))
    if handovers > 0:
        print(f"tile hand-over, mean clocks over {handovers} hand-overs: finished tile seen by the epilogue -> shared columns "
              f"in registers, accumulator released: {(released - seen) / handovers:.0f} (tcgen05 fence passed after {(fenced - seen) / handovers:.0f}, first load issued after {(first_ld - seen) / handovers:.0f}, loads issued after {(ld_issued - seen) / handovers:.0f}, "
              f"data there after {(loaded - seen) / handovers:.0f}); released -> seen by the issuer: "
              f"{(taken - released) / handovers:.0f}")
    if no_loads:
        print("producers loaded only the first fill of the ring: stage time without operand traffic into shared memory")
    stages = t[:, 3].mean().item()
    print(f"issuer clocks per K stage of 256: {total / stages:.0f} (4 MMAs of 128 clk = 512 when the tensor pipe never waits)")


if __name__ == "__main__":
    main()
