"""Timing tables for the FP4 path, after the reference's speed_test.py.

    python -m nvfp_kernel_b200.speed_test                 # BF16 torch.mm vs FP4 (online activation quantize + GEMM)
    python -m nvfp_kernel_b200.speed_test --table decode  # Llama-3-8B decode shapes, M in {1, 16, 128}
    python -m nvfp_kernel_b200.speed_test --table quant   # quantizer alone, GB/s
    python -m nvfp_kernel_b200.speed_test --table fp4out  # GEMM + quantizer of its output, separate and fused
    python -m nvfp_kernel_b200.speed_test --table mxfp4   # MXFP4 at M = 4096, K = N = 8192, beside NVFP4
    python -m nvfp_kernel_b200.speed_test --table host    # host microseconds per call (enqueue only)
    python -m nvfp_kernel_b200.speed_test --table mlp     # gated MLP: separate kernels vs activation + quantizer in the epilogue
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 -m nvfp_kernel_b200.speed_test --table tp
                                                          # Llama-3-70B prefill layers, tensor-parallel

The first table is the reference's sweep (speed_test.py:56-98 there): M = --batch_size (default 4096),
K = N = size, weight quantized once, activation amax + quantize + GEMM timed per call.  Differences:
CUDA events instead of torch.utils.benchmark, an L2 flush between timed calls, and the FP4 TFLOPS column is
computed from the FP4 time (the reference divides by the BF16 time, speed_test.py:94, so its two TFLOPS
columns are equal).
"""
from __future__ import annotations

import argparse
import statistics

import torch

from . import QuantLinear, ops

_FLUSH = None


def _flush_l2():
    global _FLUSH
    if _FLUSH is None:
        _FLUSH = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    _FLUSH.zero_()


def time_us(fn, repeats: int, flush: bool = True) -> float:
    """Median device time of fn() in microseconds (CUDA events, 5 warm-up calls)."""
    for _ in range(5):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(repeats):
        if flush:
            _flush_l2()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        e1.synchronize()
        times.append(e0.elapsed_time(e1) * 1e3)
    return statistics.median(times)


def time_us_interleaved(fns, repeats: int):
    """Median device times of several alternatives, measured in turn within every repeat: on second-long,
    power-limited work the clocks drift during a table row, and alternatives timed one after the other would not
    see the same clocks."""
    for fn in fns:
        for _ in range(5):
            fn()
    torch.cuda.synchronize()
    times = [[] for _ in fns]
    for _ in range(repeats):
        for i, fn in enumerate(fns):
            _flush_l2()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            e1.synchronize()
            times[i].append(e0.elapsed_time(e1) * 1e3)
    return [statistics.median(t) for t in times]


def _graphed(fn):
    """fn captured in a CUDA graph; returns the replay callable (decode-sized work is launch-bound otherwise)."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        fn()
    return graph.replay


def sweep(batch_size: int, repeats: int):
    print(f"{'Size (K=N)':<10} {'BF16 (us)':<12} {'FP4 (us)':<12} {'Speedup':<10} {'BF16 TFLOPS':<14} {'FP4 TFLOPS':<12}")
    print("-" * 74)
    for size in (64, 128, 256, 512, 1024, 2048, 4096, 8192):
        m, k, n = batch_size, size, size
        a = torch.randn(m, k, dtype=torch.bfloat16, device="cuda")
        w = torch.randn(n, k, dtype=torch.bfloat16, device="cuda")
        wt = w.t().contiguous()
        flops = 2.0 * m * k * n
        t_bf16 = time_us(lambda: torch.mm(a, wt), repeats)
        layer = QuantLinear(k, n, device="cuda").load_weight(w)
        t_fp4 = time_us(lambda: layer(a), repeats)
        print(f"{size:<10} {t_bf16:<12.1f} {t_fp4:<12.1f} {t_bf16 / t_fp4:<10.2f} "
              f"{flops / t_bf16 / 1e6:<14.1f} {flops / t_fp4 / 1e6:<12.1f}")


def decode(repeats: int):
    print(f"{'M':<5} {'K':<7} {'N':<7} {'bf16 mm (us)':<13} {'GEMM (us)':<11} {'GB/s':<9} {'forward (us)':<13} {'graph replay (us)':<13}")
    print("-" * 90)
    for m in (1, 16, 128):
        for k, n in ((4096, 6144), (4096, 4096), (4096, 28672), (14336, 4096), (8192, 57344)):
            a = torch.randn(m, k, dtype=torch.bfloat16, device="cuda")
            w = (torch.randn(n, k, device="cuda") * 0.02).to(torch.bfloat16)
            wt = w.t()
            t_bf16 = time_us(lambda: torch.mm(a, wt), repeats)          # the unquantized layer (cuBLAS)
            layer = QuantLinear(k, n, device="cuda").load_weight(w)
            del wt
            gs = ops.global_scale(a)
            a_fp4, a_sf = ops.scaled_fp4_quant(a, gs)
            alpha = ops.alpha_from_scales(gs, layer.weight_global_scale)
            w_sf = layer.weight_sf.view(torch.float8_e4m3fn)
            t_mm = time_us(lambda: ops.cutlass_scaled_fp4_mm(a_fp4, layer.weight_fp4, a_sf, w_sf, alpha, torch.bfloat16),
                           repeats)
            t_fwd = time_us(lambda: layer(a), repeats)
            layer.enable_cuda_graph()
            a_static = layer.graph_input(a.shape, a.dtype)     # the activation written where the graph reads it
            a_static.copy_(a)
            t_graph = time_us(lambda: layer(a_static), repeats)
            nbytes = n * k * 0.5625 + m * k * 0.5625 + 2.0 * m * n
            print(f"{m:<5} {k:<7} {n:<7} {t_bf16:<13.1f} {t_mm:<11.1f} {nbytes / t_mm / 1e3:<9.0f} {t_fwd:<13.1f} {t_graph:<13.1f}")


def host(repeats: int):
    """Host time per call (enqueue only, microseconds): how long the calling thread is busy before the call returns,
    with the GPU kept behind (bursts of calls, then a synchronize).  What a decode loop pays per layer on the CPU."""
    import time
    print(f"{'M':<5} {'K':<7} {'N':<7} {'GEMM call (us)':<16} {'forward call (us)':<18} {'C ABI GEMM (us)':<16}")
    print("-" * 72)
    from . import _capi
    lib = _capi.load()
    for m, k, n in ((16, 4096, 4096), (16, 4096, 28672), (128, 4096, 6144), (2048, 4096, 4096)):
        a = torch.randn(m, k, dtype=torch.bfloat16, device="cuda")
        w = (torch.randn(n, k, device="cuda") * 0.02).to(torch.bfloat16)
        layer = QuantLinear(k, n, device="cuda").load_weight(w)
        gs = ops.global_scale(a)
        a_fp4, a_sf = ops.scaled_fp4_quant(a, gs)
        alpha = ops.alpha_from_scales(gs, layer.weight_global_scale)
        w_sf = layer.weight_sf.view(torch.float8_e4m3fn)
        out = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
        stream = torch.cuda.current_stream().cuda_stream
        args = (out.data_ptr(), a_fp4.data_ptr(), layer.weight_fp4.data_ptr(), a_sf.data_ptr(), layer.weight_sf.data_ptr(),
                alpha.data_ptr(), m, n, k, _capi.NVFP_DTYPE_BF16, stream)

        def burst(fn, calls=64):
            best = float("inf")
            for _ in range(max(3, repeats // 8)):
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                for _ in range(calls):
                    fn()
                best = min(best, (time.perf_counter() - t0) / calls * 1e6)
            torch.cuda.synchronize()
            return best

        t_mm = burst(lambda: ops.cutlass_scaled_fp4_mm(a_fp4, layer.weight_fp4, a_sf, w_sf, alpha, torch.bfloat16))
        t_fwd = burst(lambda: layer(a))
        t_c = burst(lambda: lib.nvfp_scaled_fp4_mm(*args))
        print(f"{m:<5} {k:<7} {n:<7} {t_mm:<16.1f} {t_fwd:<18.1f} {t_c:<16.1f}")


def quant(repeats: int):
    print(f"{'M':<7} {'K':<7} {'quantize (us)':<15} {'GB/s (2.5625 B/elt)':<20} {'amax (us)':<10}")
    print("-" * 62)
    for m, k in ((1, 4096), (128, 4096), (4096, 4096), (8192, 8192), (8192, 28672)):
        a = torch.randn(m, k, dtype=torch.bfloat16, device="cuda")
        gs = ops.global_scale(a)
        t_q = time_us(lambda: ops.scaled_fp4_quant(a, gs), repeats)
        t_a = time_us(lambda: ops.global_scale(a), repeats)
        print(f"{m:<7} {k:<7} {t_q:<15.1f} {m * k * 2.5625 / t_q / 1e3:<20.0f} {t_a:<10.1f}")


def mxfp4(repeats: int):
    """MXFP4 (32-element blocks, ue8m0 scales, no global scale) at M = 4096, K = N = 8192: Student-t (df = 3)
    activations, N(0, 0.02) weights; the NVFP4 numbers of the same shape beside them."""
    m, k, n = 4096, 8192, 8192
    g = torch.Generator(device="cuda").manual_seed(0)
    z = torch.randn((m, k), generator=g, device="cuda")
    chi = sum(torch.randn((m, k), generator=g, device="cuda") ** 2 for _ in range(3)) / 3.0
    a = (z / chi.sqrt()).to(torch.bfloat16)
    w = (torch.randn((n, k), generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    del z, chi
    print(f"{'format':<8} {'quantize A (us)':<17} {'GB/s':<8} {'GEMM (us)':<11} {'TFLOP/s':<9} {'forward (us)':<13}")
    print("-" * 70)
    for fmt in ("mxfp4", "nvfp4"):
        layer = QuantLinear(k, n, format=fmt, device="cuda").load_weight(w)
        if fmt == "mxfp4":
            a_fp4, a_sf = ops.scaled_mxfp4_quant(a)
            w_sf = layer.weight_sf.view(torch.float8_e8m0fnu)
            t_q = time_us(lambda: ops.scaled_mxfp4_quant(a), repeats)
            t_mm = time_us(lambda: ops.mxfp4_scaled_mm(a_fp4, layer.weight_fp4, a_sf, w_sf, torch.bfloat16), repeats)
            bytes_per = 2.0 + 0.5 + 1.0 / 32
        else:
            gs = ops.global_scale(a)
            a_fp4, a_sf = ops.scaled_fp4_quant(a, gs)
            alpha = ops.alpha_from_scales(gs, layer.weight_global_scale)
            w_sf = layer.weight_sf.view(torch.float8_e4m3fn)
            t_q = time_us(lambda: ops.scaled_fp4_quant(a, gs), repeats)
            t_mm = time_us(lambda: ops.cutlass_scaled_fp4_mm(a_fp4, layer.weight_fp4, a_sf, w_sf, alpha, torch.bfloat16), repeats)
            bytes_per = 2.5625
        t_fwd = time_us(lambda: layer(a), repeats)
        print(f"{fmt:<8} {t_q:<17.1f} {m * k * bytes_per / t_q / 1e3:<8.0f} {t_mm:<11.1f} {2.0 * m * n * k / t_mm / 1e6:<9.0f} {t_fwd:<13.1f}")


def fp4out(repeats: int):
    """A layer whose output feeds another NVFP4 layer: GEMM -> bf16 tensor -> global scale -> quantizer, against the
    GEMM that quantizes in its epilogue (output scale known beforehand)."""
    print(f"{'M':<6} {'K':<6} {'N':<6} {'GEMM (us)':<11} {'+ amax + quantize (us)':<24} {'GEMM with NVFP4 output (us)':<28}")
    print("-" * 84)
    for m, k, n in ((8192, 8192, 8192), (4096, 4096, 4096), (8192, 8192, 28672), (2048, 4096, 14336)):
        a = torch.randn(m, k, dtype=torch.bfloat16, device="cuda")
        w = (torch.randn(n, k, device="cuda") * 0.02).to(torch.bfloat16)
        ga, gw = ops.global_scale(a), ops.global_scale(w)
        a_fp4, a_sf = ops.scaled_fp4_quant(a, ga)
        w_fp4, w_sf = ops.scaled_fp4_quant(w, gw)
        del a, w
        alpha = ops.alpha_from_scales(ga, gw)
        out_gs = ops.global_scale(ops.cutlass_scaled_fp4_mm(a_fp4, w_fp4, a_sf, w_sf, alpha, torch.bfloat16))

        def separate():
            y = ops.cutlass_scaled_fp4_mm(a_fp4, w_fp4, a_sf, w_sf, alpha, torch.bfloat16)
            return ops.scaled_fp4_quant(y, ops.global_scale(y))

        t_mm = time_us(lambda: ops.cutlass_scaled_fp4_mm(a_fp4, w_fp4, a_sf, w_sf, alpha, torch.bfloat16), repeats)
        t_sep = time_us(separate, repeats)
        t_fused = time_us(lambda: ops.scaled_fp4_mm_fp4out(a_fp4, w_fp4, a_sf, w_sf, alpha, out_gs), repeats)
        print(f"{m:<6} {k:<6} {n:<6} {t_mm:<11.1f} {t_sep:<24.1f} {t_fused:<28.1f}")


def mlp(repeats: int):
    """Gated MLP (Llama shapes) from a bf16 activation to a bf16 result: every step a separate kernel, against the
    gate/up GEMM that applies silu(gate) * up and quantizes for the down projection in its epilogue, and against
    the same three kernels issued by one call and chained with programmatic dependent launch (what QuantGatedMLP
    runs).  Rows of 128 tokens or fewer are timed as CUDA graph replays."""
    import torch.nn.functional as F
    print(f"{'model':<12} {'M':<6} {'hidden':<7} {'inter':<7} {'separate (us)':<15} {'fused epilogue (us)':<21} "
          f"{'one call, chained (us)':<24} {'TFLOP/s':<8}")
    print("-" * 106)
    for name, m, hidden, inter in (("llama-3-8b", 8192, 4096, 14336), ("llama-3-70b", 8192, 8192, 28672),
                                   ("llama-3-8b", 512, 4096, 14336), ("llama-3-8b", 128, 4096, 14336),
                                   ("llama-3-8b", 16, 4096, 14336), ("llama-3-70b", 16, 8192, 28672)):
        x = torch.randn(m, hidden, dtype=torch.bfloat16, device="cuda")
        w_gu = (torch.randn(2 * inter, hidden, device="cuda") * 0.02).to(torch.bfloat16)   # already interleaved
        w_d = (torch.randn(hidden, inter, device="cuda") * 0.02).to(torch.bfloat16)
        ggu, gd = ops.global_scale(w_gu), ops.global_scale(w_d)
        gu_fp4, gu_sf = ops.scaled_fp4_quant(w_gu, ggu)
        d_fp4, d_sf = ops.scaled_fp4_quant(w_d, gd)
        del w_gu, w_d
        scratch = torch.zeros(8, dtype=torch.int32, device="cuda")

        def separate():
            x_fp4, x_sf, _, alpha1 = ops.dynamic_scaled_fp4_quant(x, scratch, ggu)
            y = ops.cutlass_scaled_fp4_mm(x_fp4, gu_fp4, x_sf, gu_sf, alpha1, torch.bfloat16).view(m, inter // 16, 2, 16)
            h = F.silu(y[:, :, 0]) * y[:, :, 1]
            h_fp4, h_sf, _, alpha2 = ops.dynamic_scaled_fp4_quant(h.view(m, inter), scratch, gd)
            return ops.cutlass_scaled_fp4_mm(h_fp4, d_fp4, h_sf, d_sf, alpha2, torch.bfloat16)

        separate()
        gh = ops.global_scale((F.silu(torch.randn(m, 64, device="cuda")) * torch.randn(m, 64, device="cuda")).to(torch.bfloat16))
        alpha2 = ops.alpha_from_scales(gh, gd)                 # calibrated scale of the hidden activation

        def fused():
            x_fp4, x_sf, _, alpha1 = ops.dynamic_scaled_fp4_quant(x, scratch, ggu)
            h_fp4, h_sf = ops.scaled_fp4_mm_silu_mul(x_fp4, gu_fp4, x_sf, gu_sf, alpha1, torch.bfloat16, out_global_scale=gh)
            return ops.cutlass_scaled_fp4_mm(h_fp4, d_fp4, h_sf, d_sf, alpha2, torch.bfloat16)

        def chained():
            return ops.gated_mlp_forward(x, gu_fp4, gu_sf, ggu, d_fp4, d_sf, gh, alpha2, scratch, torch.bfloat16)

        if m <= 128:
            separate, fused, chained = _graphed(separate), _graphed(fused), _graphed(chained)
        t_sep, t_fused, t_chain = time_us_interleaved((separate, fused, chained), repeats)
        flops = 2.0 * m * hidden * inter * 3
        print(f"{name:<12} {m:<6} {hidden:<7} {inter:<7} {t_sep:<15.1f} {t_fused:<21.1f} {t_chain:<24.1f} "
              f"{flops / t_chain / 1e6:<8.0f}")
        del gu_fp4, gu_sf, d_fp4, d_sf, x
        torch.cuda.empty_cache()


def tensor_parallel(repeats: int):
    """Llama-3-70B prefill layers (M = 8192) sharded over the ranks of this launch (torchrun):
    gate_up [N = 57344, K = 8192] column-parallel, down [N = 8192, K = 28672] row-parallel, each with the
    NCCL collective after the GEMM and with the collective fused into the GEMM epilogue.  Every rank builds
    only its own weight shard (random values: this table times, the tests check values)."""
    import os
    import torch.distributed as dist
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    m = 8192
    g = torch.Generator(device="cuda").manual_seed(0)

    def timed(layer, x):
        for _ in range(3):
            layer(x)
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(repeats):
            layer(x)
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / repeats], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    def make(parallel, n, k, **kw):
        layer = QuantLinear(k, n, parallel=parallel, device="cuda", **kw)
        shard = (torch.randn((layer.n_local, layer.k_local), generator=g, device="cuda") * 0.02).to(torch.bfloat16)
        gs = ops.global_scale(shard)
        w_fp4, w_sf = ops.scaled_fp4_quant(shard, gs)
        layer.weight_fp4, layer.weight_sf = w_fp4, w_sf.view(torch.uint8)
        layer.weight_global_scale.copy_(gs)
        return layer

    rows = []
    x = torch.randn((m, 8192), generator=g, device="cuda").to(torch.bfloat16)
    flops = 2.0 * m * 57344 * 8192
    for name, kw in (("NCCL all-gather", {}), ("fused gather", {"fused_gather": True})):
        if world == 1 and kw:
            continue
        t = timed(make("column" if world > 1 else None, 57344, 8192, **kw), x)
        rows.append(("gate_up column-parallel", name if world > 1 else "single GPU", t, flops / t / 1e9))
    x = torch.randn((m, 28672), generator=g, device="cuda").to(torch.bfloat16)
    flops = 2.0 * m * 8192 * 28672
    for name, kw in (("NCCL reduce-scatter", {}), ("fused reduce-scatter", {"fused_reduce_scatter": True})):
        if world == 1 and kw:
            continue
        t = timed(make("row" if world > 1 else None, 8192, 28672, **kw), x)
        rows.append(("down row-parallel", name if world > 1 else "single GPU", t, flops / t / 1e9))
    # the whole gated MLP, intermediate dimension split: quantize, gate/up GEMM (silu * up and NVFP4 quantization in the
    # epilogue), down GEMM with its partial sums reduce-scattered; every rank builds only its own shards
    from . import QuantGatedMLP
    x = torch.randn((m, 8192), generator=g, device="cuda").to(torch.bfloat16)
    flops = 2.0 * m * 8192 * 28672 * 3
    for name, kw in (("NCCL reduce-scatter", {}), ("fused reduce-scatter", {"fused_reduce_scatter": True})):
        if world == 1 and kw:
            continue
        mlp_layer = QuantGatedMLP(8192, 28672, parallel="tensor" if world > 1 else None, device="cuda", **kw)
        il = mlp_layer.inter_local
        for w_name, sf_name, gs_name, shape in (("gate_up_fp4", "gate_up_sf", "gate_up_global_scale", (2 * il, 8192)),
                                                ("down_fp4", "down_sf", "down_global_scale", (8192, il))):
            shard = (torch.randn(shape, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
            gs = ops.global_scale(shard)
            w_fp4, w_sf = ops.scaled_fp4_quant(shard, gs)
            setattr(mlp_layer, w_name, w_fp4)
            setattr(mlp_layer, sf_name, w_sf.view(torch.uint8))
            getattr(mlp_layer, gs_name).copy_(gs)
            del shard
        mlp_layer.set_activation_scale(torch.tensor([2688.0 / 4.0], device="cuda"))
        t = timed(mlp_layer, x)
        rows.append(("gated MLP tensor-parallel", name if world > 1 else "single GPU", t, flops / t / 1e9))
        del mlp_layer
        torch.cuda.empty_cache()
    if rank == 0:
        print(f"Llama-3-70B prefill layers, M = {m}, {world} GPU(s); time = max over ranks, includes activation quantize")
        print(f"{'layer':<26} {'collective':<22} {'ms':<9} {'TFLOP/s (all ranks)':<20}")
        for r in rows:
            print(f"{r[0]:<26} {r[1]:<22} {r[2]:<9.3f} {r[3]:<20.0f}")
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser(description="BF16 GEMM vs FP4 GEMM with online activation quantization")
    ap.add_argument("--batch_size", type=int, default=4096, help="M dimension of the sweep")
    ap.add_argument("--repeats", type=int, default=50)
    ap.add_argument("--table", default="sweep", choices=["sweep", "decode", "quant", "tp", "fp4out", "mlp", "mxfp4", "host"])
    args = ap.parse_args()
    torch.cuda.empty_cache()
    {"sweep": lambda: sweep(args.batch_size, args.repeats), "decode": lambda: decode(args.repeats),
     "quant": lambda: quant(args.repeats), "host": lambda: host(args.repeats), "fp4out": lambda: fp4out(min(args.repeats, 20)), "mlp": lambda: mlp(min(args.repeats, 10)), "mxfp4": lambda: mxfp4(min(args.repeats, 20)), "tp": lambda: tensor_parallel(min(args.repeats, 20))}[args.table]()


if __name__ == "__main__":
    main()
