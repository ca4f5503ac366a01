#!/usr/bin/env python
"""Benchmark of the NVFP4 hot path: activation amax + quantize -> block-scaled FP4 GEMM.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--gather fused|nccl]

One step = one forward of QuantLinear(mode="real") on M=N=K=8192 (per GPU): global scale
of the bf16 activation, NVFP4 quantize, alpha, FP4 GEMM with bf16 output (the flow of the
reference's speed_test.py:36-50; the weight is quantized once, outside the timed region).
With N>1 the layer is column-parallel: every rank holds 8192 output columns (weak scaling)
and the step ends with the all-gather of the bf16 outputs.

Prints ONE JSON line (rank 0).
  value      2*M*N_total*K / step time in TFLOP/s over exactly --steps steps, activation resident in HBM (a burst:
             a few milliseconds at full clock)
  sustained  the same step repeated for at least a second (the 1000 W cap engages), with the GEMM kernel timed
             inside such a run, the SM clock seen and time x clock
  e2e        the same through the public Python API with the activation in pinned host memory and the output
             copied back, every step
  roofline   the GEMM kernel timed alone inside the run with CUDA events
  parity     (N > 1) the fused gather compared bitwise with the NCCL all-gather of the same layer, this rank's slab
             against the exact product of the bytes it consumed, and the row-parallel fused reduce-scatter of the
             Llama-3-70B down projection against NCCL reduce_scatter of the fp32 partial products; the run exits
             non-zero when one of them fails
  extra      the two Llama-3-70B prefill layers (gate_up column-parallel, down row-parallel) at this N
  cpu_baseline  the CPU port of the reference's torch pseudo-quant path on a bounded sample (N = 1)

`--impl reference` times that CPU path alone (the reference has no kernel that can run on
sm_100: its GEMM is a CUTLASS sm_120a instantiation).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

M = N_PER_GPU = K = 8192
C4_GATE_UP_N, C4_DOWN_K = 57344, 28672          # Llama-3-70B prefill layers (hidden 8192)
METRIC = "nvfp4_gemm_tflops_m8192_n8192_k8192"
NOMINAL_FP4_TFLOPS = 9000.0
NOMINAL_HBM_GBS = 8000.0
# DRAM bytes the GEMM launch of this workload moved under ncu (101.7 MB read + 110.0 MB written in the latest capture:
# both operands and their scales read once; of the 134 MB of output, 110 MB reached DRAM before the kernel ended, the
# rest sat in L2).
GEMM_DRAM_BYTES_PER_LAUNCH = 211.7e6
# operands (2 x M*K/2) + scales (2 x M*K/16) + bf16 output
GEMM_ALGORITHMIC_BYTES = 2 * (M * K // 2) + 2 * (M * K // 16) + 2 * M * N_PER_GPU


def load_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
                "source": "measured"}
    except Exception:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def workload_config(world: int, gather: str) -> dict:
    """`config` of the JSON line; the same for both arms (the reference arm adds its row sample)."""
    return {
        "workload": f"nvfp4_quant_linear_M{M}_N{N_PER_GPU}x{world}_K{K}",
        "step": "amax -> global scale and alpha (one kernel), NVFP4 quantize of the bf16 activation, FP4 GEMM, bf16 out"
                + (", all-gather of outputs (column-parallel)" if world > 1 else ""),
        "parallelism": (f"column-parallel x{world}, gather " + {
            "fused": "fused into the GEMM epilogue (peer stores)", "nccl": "by NCCL all-gather",
            "fused-fp4": "of the NVFP4 form of the output, fused into the GEMM epilogue (peer stores)"}[gather])
        if world > 1 else "single GPU",
        "l2": "no flush: bf16 activation (134 MB) + output (134 MB) per step exceed the 126 MB L2",
    }


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while a region runs."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    def _run(self):
        nv = self._nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                get = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                    nv.nvmlDeviceGetCurrentClocksThrottleReasons
                mask = get(self._h)
                for k, bit in names.items():
                    if mask & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(0.005)

    def __enter__(self):
        if self._nv is not None:
            self._stop.clear()
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        if self._thread is not None:
            self._stop.set()
            self._thread.join()
            self._thread = None

    def fork(self) -> "ClockSampler":
        """A sampler for another region of the same run (own samples, same NVML handle)."""
        other = ClockSampler.__new__(ClockSampler)
        other.samples, other.reasons, other.max_mhz = [], set(), self.max_mhz
        other._stop, other._thread = threading.Event(), None
        other._nv = self._nv
        if self._nv is not None:
            other._h = self._h
        return other

    def summary(self):
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ------------------------------------------------------------------ CPU reference arm ---
def cpu_reference_step_factory(seed: int = 0):
    """Weight side done once (offline, like the reference flow); returns step(rows) which runs
    the activation side of the reference's pseudo-quant path on `rows` rows and the float64
    matmul against the full dequantized weight."""
    from oracle import pseudo_path
    g = torch.Generator().manual_seed(seed + 1)
    w = torch.randn((N_PER_GPU, K), generator=g, dtype=torch.float32).to(torch.bfloat16)
    w_dq_t = pseudo_path.dequantize(*pseudo_path.quantize(w)).T.contiguous()
    g = torch.Generator().manual_seed(seed)
    a_full = torch.randn((1024, K), generator=g, dtype=torch.float32).to(torch.bfloat16)

    def step(rows: int) -> float:
        a = a_full[:rows]
        t0 = time.perf_counter()
        y = pseudo_path.dequantize(*pseudo_path.quantize(a)) @ w_dq_t
        dt = time.perf_counter() - t0
        assert y.shape == (rows, N_PER_GPU)
        return dt

    return step


def run_cpu_baseline(budget_s: float, steps: int, warmup: int):
    """Returns (TFLOP/s, threads used, sample description, ms per step, rows per step).  Uses every host core this
    process may run on: a launcher such as torch.distributed.run exports OMP_NUM_THREADS=1, which would otherwise
    leave the CPU arm on one thread."""
    threads = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    torch.set_num_threads(max(1, threads))
    step = cpu_reference_step_factory()
    t_probe = step(64)
    rows = int(max(16, min(1024, (budget_s / max(1, steps + warmup)) / (t_probe / 64))) // 16 * 16)
    for _ in range(warmup):
        step(rows)
    times = [step(rows) for _ in range(steps)]
    t = sum(times) / len(times)
    tflops = 2.0 * rows * N_PER_GPU * K / t / 1e12
    sample = (f"{rows} of {M} activation rows per step (quantize + dequantize + float64 matmul against the full "
              f"[{N_PER_GPU},{K}] dequantized weight; weight side prepared once, untimed), mean of {steps} steps, "
              f"{torch.get_num_threads()} threads")
    return tflops, torch.get_num_threads(), sample, t * 1e3, rows


def main_reference(args, rank: int):
    if rank != 0:
        return
    tflops, cores, sample, ms, rows = run_cpu_baseline(120.0, args.steps, args.warmup)
    config = workload_config(args.gpus, args.gather)
    config["cpu_rows_per_step"] = rows
    config["note"] = ("CPU port of the reference's torch pseudo-quant path (the reference's CUDA GEMM is sm_120a-only "
                      "and cannot run on B200); each step is a bounded row sample of the workload, quoted as a rate")
    line = {
        "impl": "reference", "metric": METRIC, "value": tflops, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f64", "data": "synthetic", "config": config,
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------- GPU arm ---
def dequantize_fp32(packed: torch.Tensor, sf_swizzled: torch.Tensor) -> torch.Tensor:
    """NVFP4 bytes -> value * block scale as fp32 [rows, k] (exact: 6 significant bits at most)."""
    rows, kh = packed.shape
    k = kh * 2
    lut = torch.tensor([0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6], dtype=torch.float32,
                       device=packed.device)
    vals = torch.stack((lut[(packed & 0xF).long()], lut[(packed >> 4).long()]), dim=-1).reshape(rows, k // 16, 16)
    rp, cp = sf_swizzled.shape
    sf = sf_swizzled.view(torch.uint8).reshape(rp // 128, cp // 4, 32, 4, 4).transpose(1, 3).reshape(rp, cp)[:rows, :k // 16]
    return (vals * sf.contiguous().view(torch.float8_e4m3fn).float().unsqueeze(-1)).reshape(rows, k)


def gemm_tolerance(out: torch.Tensor, ref: torch.Tensor, rel: float = 1e-2):
    """The GEMM contract: max|out-ref| <= rel*max|ref| and per element |out-ref| <= rel*|ref| + 2^-8*rms(ref).
    Returns (passed, max|out-ref| / max|ref|)."""
    out, ref = out.float(), ref.float()
    err = (out - ref).abs()
    mx = ref.abs().max()
    rms = ref.pow(2).mean().sqrt()
    ok = bool(torch.isfinite(out).all()) and bool(err.max() <= rel * mx) and \
        not bool((err > rel * ref.abs() + rms * 2.0 ** -8).any())
    return ok, float(err.max() / mx)


def main_ours(args, rank: int, world: int, local_rank: int):
    import torch.distributed as dist
    import nvfp_kernel_b200 as nv
    from nvfp_kernel_b200 import QuantLinear

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    peaks = load_peaks()
    n_total = N_PER_GPU * world
    fused = args.gather != "nccl"
    fp4_gather = args.gather == "fused-fp4" and world > 1
    own_launches = [0]          # this package's kernels launched inside timed regions (counted per call below)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def all_ranks(flag: bool) -> bool:
        if world == 1:
            return flag
        t = torch.tensor([1 if flag else 0], device=dev, dtype=torch.int32)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return bool(t.item())

    def global_weight_scale(w_local):
        """One global scale for the whole (sharded) weight, as a 1-GPU layer would use."""
        amax = w_local.float().abs().max().reshape(1)
        if world > 1:
            dist.all_reduce(amax, op=dist.ReduceOp.MAX)
        return (2688.0 / amax).to(torch.float32)

    def install_weight(layer, w_local):
        gs_w = global_weight_scale(w_local)
        w_fp4, w_sf = nv.scaled_fp4_quant(w_local, gs_w)
        layer.weight_fp4, layer.weight_sf = w_fp4, w_sf.view(torch.uint8)
        layer.weight_global_scale.copy_(gs_w)
        return layer

    def randn_bf16(shape, seed, std=1.0):
        g = torch.Generator(device=dev).manual_seed(seed)
        return (torch.randn(shape, generator=g, device=dev, dtype=torch.float32) * std).to(torch.bfloat16)

    def timed(fn, steps: int, launches_per_call: int):
        """ms per call over exactly `steps` calls: barrier + synchronize on both sides, CUDA events, max over ranks."""
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        own_launches[0] += steps * launches_per_call
        return max_over_ranks(e0.elapsed_time(e1) / steps)

    # synthetic data: activations ~N(0,1) (same on every rank), weights ~N(0,1) as in the
    # reference's speed_test.py:74-75; each rank draws only its own 8192 output columns
    a = randn_bf16((M, K), 0)
    if world > 1:
        # this rank's column slab of a column-parallel layer; the gather is fused into the GEMM epilogue
        # (peer stores over NVLink) unless --gather nccl asks for the all-gather collective
        layer = QuantLinear(K, n_total, parallel="column", fused_gather=fused, device=dev)
    else:
        layer = QuantLinear(K, N_PER_GPU, device=dev)
    install_weight(layer, randn_bf16((N_PER_GPU, K), 1000 + rank))
    # in-kernel waits on peer ranks: the library's bound is two seconds; the processes of a benchmark start their
    # first calls with whatever skew the host gives them, so allow the maximum (ten seconds) here
    PEER_WAIT_NS = 10_000_000_000
    layer.peer_wait_limit_ns = PEER_WAIT_NS
    gathered = torch.empty((world * M, N_PER_GPU), dtype=torch.bfloat16, device=dev) if world > 1 else None
    layer.gather_output = fused

    fp4_out_gs = [None]                  # calibrated global scale of the gathered output (NVFP4 gather only)

    def step_bf16(x):
        y = layer(x)                     # fused gather: already the full [M, n_total] matrix
        if world > 1 and not fused:
            dist.all_gather_into_tensor(gathered, y)     # layout [world, M, N/world]
            return gathered
        return y

    def step(x):
        if fp4_gather and fp4_out_gs[0] is not None:
            return layer.forward_gather_fp4(x, fp4_out_gs[0])[0]      # gathered NVFP4 operand (packed bytes)
        return step_bf16(x)

    sampler = ClockSampler(local_rank)
    launches_per_step = 3 if world == 1 or fused else 4   # amax(+scales), quantize, gemm (+ all-gather)
    own_kernels_per_step = 3
    warmup = max(3, args.warmup)
    for _ in range(warmup):
        step(a)
    barrier()

    # ---- parity (N > 1), outside every timed region ------------------------------------------------------------
    parity = None
    if world > 1:
        parity = {}
        y_gathered = step_bf16(a)
        if not fused:
            y_gathered = y_gathered.view(world, M, N_PER_GPU).permute(1, 0, 2).reshape(M, n_total)
        y_gathered = y_gathered.clone()
        # (a) the same layer through the other gather: bitwise equal
        other = QuantLinear(K, n_total, parallel="column", fused_gather=not fused, device=dev)
        other.weight_fp4, other.weight_sf = layer.weight_fp4, layer.weight_sf
        other.weight_global_scale.copy_(layer.weight_global_scale)
        other.peer_wait_limit_ns = PEER_WAIT_NS
        y_other = other(a)
        column_ok = all_ranks(bool(torch.equal(y_gathered, y_other)))
        parity["column_fused_vs_nccl"] = "bitwise" if column_ok else "MISMATCH"
        del y_other, other
        # this rank's slab against the exact product of the bytes the kernel consumed (unrounded fp32)
        a_fp4, a_sf, alpha = layer._quantize_activation(a)
        ref = (dequantize_fp32(a_fp4, a_sf) @ dequantize_fp32(layer.weight_fp4, layer.weight_sf).T) * alpha
        slab_ok, slab_rel = gemm_tolerance(y_gathered[:, rank * N_PER_GPU:(rank + 1) * N_PER_GPU], ref)
        parity["own_slab_max_rel"] = max_over_ranks(slab_rel)
        slab_ok = all_ranks(slab_ok)
        # (c) the gather of the NVFP4 form of the output (quantized in the GEMM epilogue, 0.5625 B per element over
        # NVLink): bytes and scales of the gathered operand equal the quantizer's on the gathered bf16 matrix
        out_gs = (2688.0 / y_gathered.abs().max().float()).reshape(1)
        want_fp4, want_sf = nv.scaled_fp4_quant(y_gathered, out_gs)
        got_fp4, got_sf = layer.forward_gather_fp4(a, out_gs)
        fp4_ok = all_ranks(bool(torch.equal(got_fp4, want_fp4)) and
                           bool(torch.equal(got_sf.view(torch.uint8), want_sf.view(torch.uint8))))
        parity["fp4_gather_vs_quantizer_on_bf16_gather"] = "bitwise" if fp4_ok else "MISMATCH"
        fp4_out_gs[0] = out_gs
        del ref, y_gathered, a_fp4, a_sf, want_fp4, want_sf, got_fp4, got_sf
        torch.cuda.empty_cache()
        for _ in range(3):
            layer.forward_gather_fp4(a, out_gs)
        ms_fp4_gather = timed(lambda: layer.forward_gather_fp4(a, out_gs), args.steps, own_kernels_per_step)

    # ---- what NVLink gives a kernel's stores into a peer's memory on this box (N > 1): the roofline of the gather ---
    nvlink = None
    if world > 1:
        import torch.distributed._symmetric_memory as symm_mem
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        probe = symm_mem.empty((M * N_PER_GPU,), dtype=torch.bfloat16, device=dev)
        handle = symm_mem.rendezvous(probe, dist.group.WORLD)
        peer_view = handle.get_buffer((rank + 1) % world, (M * N_PER_GPU,), torch.bfloat16)
        src = torch.zeros_like(probe)
        for _ in range(2):
            peer_view.copy_(src)
        ms_copy = timed(lambda: peer_view.copy_(src), 10, 0)
        nvlink = {"peer_store_gbs": M * N_PER_GPU * 2 / (ms_copy * 1e-3) / 1e9,
                  "what": "134 MB copied by a torch elementwise kernel (SM stores) from this rank's memory into the next "
                          "rank's peer-mapped buffer, all ranks at once (a ring), max over ranks; per direction per GPU"}
        del probe, handle, peer_view, src
        torch.cuda.empty_cache()

    # ---- region 1: whole hot path, activation resident in HBM, exactly --steps steps (burst) -------------------
    with sampler:
        ms_step = timed(lambda: step(a), args.steps, own_kernels_per_step)
    flops_step = 2.0 * M * n_total * K
    value = flops_step / (ms_step * 1e-3) / 1e12

    if args.profile_mode:
        # for profiler captures: the warm-up and the burst region only, so that a capture ends quickly
        if rank == 0:
            print(json.dumps({"profile_mode": True, "ms_per_step": ms_step, "value": value, "n_gpus": world}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- region 2: the same steps with an event pair around ONE of the kernels (kernel breakdown) ---
    # calls the same ops QuantLinear.forward makes, one by one; three passes, each timing one kernel of every step
    # (a pair of events around every kernel of a step would put six event records, and their gaps, into each step)
    w_sf = layer.weight_sf.view(torch.float8_e4m3fn)

    def timed_pass(which: int, ks: int) -> float:
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(ks)]
        barrier()
        for i in range(ks):
            # the host enqueues ahead of the GPU, so no launch gap falls inside a window
            if which == 0:
                ev[i][0].record()
            a_gs, alpha = nv.activation_scales(a, layer.weight_global_scale, layer._scale_scratch)
            if which == 0:
                ev[i][1].record()
            if which == 1:
                ev[i][0].record()
            a_fp4, a_sf = nv.scaled_fp4_quant(a, a_gs)
            if which == 1:
                ev[i][1].record()
            if which == 2:
                ev[i][0].record()
            nv.cutlass_scaled_fp4_mm(a_fp4, layer.weight_fp4, a_sf, w_sf, alpha, torch.bfloat16)   # local slab only
            if which == 2:
                ev[i][1].record()
        barrier()
        own_launches[0] += 3 * ks
        return statistics.mean(e0.elapsed_time(e1) for e0, e1 in ev)

    ks = min(args.steps, 200)
    with sampler:
        t_amax, t_quant, t_gemm = timed_pass(0, ks), timed_pass(1, ks), timed_pass(2, ks)
    # ---- region 2b: the same step for at least a second: the power cap engages, the clock settles -------------
    sustained_sampler = sampler.fork()
    sustained_steps = int(min(20000, max(args.steps, 1.2 / (ms_step * 1e-3))))
    with sustained_sampler:
        ms_sustained = timed(lambda: step(a), sustained_steps, own_kernels_per_step)

    # the GEMM inside a run of at least a second (sustained clock)
    with sustained_sampler:
        t_gemm_sustained = timed_pass(2, int(min(8000, max(ks, 1.2 / (ms_step * 1e-3)))))
    gemm_tflops = 2.0 * M * N_PER_GPU * K / (t_gemm * 1e-3) / 1e12
    gemm_tflops_sustained = 2.0 * M * N_PER_GPU * K / (t_gemm_sustained * 1e-3) / 1e12
    quant_bytes = M * K * 2.5625
    quant_gbs = quant_bytes / (t_quant * 1e-3) / 1e9
    amax_gbs = M * K * 2.0 / (t_amax * 1e-3) / 1e9

    # ---- region 3: end to end through the public API with host buffers -----------------
    # The activation lives in pinned host memory.  Every step copies it to the GPUs once: each rank copies its 1/N of
    # the rows over PCIe and the ranks all-gather the pieces over NVLink (one GPU: the whole activation).  Every rank
    # ends a step holding the whole gathered [M, n_total] result; the host needs it once, so each rank copies out its
    # own [M, N_PER_GPU] column slab (all ranks together: the whole result, every step).
    rows_per_rank = M // world
    a_host = a[rank * rows_per_rank:(rank + 1) * rows_per_rank].cpu().pin_memory()
    out_host = torch.empty((M * N_PER_GPU,), dtype=torch.bfloat16).pin_memory()
    a_part = torch.empty_like(a[:rows_per_rank])
    a_full = torch.empty_like(a)
    e2e_steps = max(3, min(args.steps, 20))

    def step_for_host(x_part):
        if world > 1:
            dist.all_gather_into_tensor(a_full, x_part)
            x = a_full
        else:
            x = x_part
        y = step_bf16(x)                                         # the host receives bf16 in every mode
        if world == 1:
            return y
        if not fused:
            return y.view(world, M, N_PER_GPU)[rank]            # all_gather_into_tensor's layout: [world, M, N/world]
        return y[:, rank * N_PER_GPU:(rank + 1) * N_PER_GPU]     # this rank's columns of the gathered matrix

    def e2e_step():
        a_part.copy_(a_host, non_blocking=True)
        y = step_for_host(a_part)
        out_host.copy_(y.reshape(-1), non_blocking=True)

    for _ in range(2):
        e2e_step()
    with sampler:
        ms_e2e_serial = timed(e2e_step, e2e_steps, own_kernels_per_step)

    # the same calls through HostPipeline: the copy-in of step i+1, the kernels of step i and the copy-out of step
    # i-1 run at the same time (PCIe is full duplex); every step still copies its own input in and its result out
    pipe = nv.HostPipeline(step_for_host, depth=2, device=dev, reuses_output=world > 1)
    out_hosts = [out_host, torch.empty_like(out_host).pin_memory()]
    for i in range(3):
        pipe.submit(a_host, out_hosts[i % 2])
    pipe.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with sampler:
        barrier()
        e0.record(pipe.copy_in)
        for i in range(e2e_steps):
            pipe.submit(a_host, out_hosts[i % 2])
        e1.record(pipe.copy_out)
        pipe.synchronize()
        barrier()
    own_launches[0] += own_kernels_per_step * e2e_steps
    ms_e2e = max_over_ranks(e0.elapsed_time(e1) / e2e_steps)
    e2e_value = flops_step / (ms_e2e * 1e-3) / 1e12
    del pipe, a_full, a_part

    # ---- extra: the Llama-3-70B prefill layers of the reference's tensor-parallel configuration -------------------
    # gate_up [57344, 8192] column-parallel (N split, outputs gathered), down [8192, 28672] row-parallel (K split,
    # partial products reduce-scattered over the rows); activations ~N(0,1) with 1 % of the K channels x50, weights
    # ~N(0, 0.02^2).  Weak-scaling layer `layer` and its buffers are released first.
    extra = {}
    if world == 1:
        # two such layers in a row: layer 1's GEMM forms the global scale of its output in its epilogue, so layer 2
        # skips its pass over the activation for the maximum (quantize -> GEMM only)
        layer2 = install_weight(QuantLinear(N_PER_GPU, N_PER_GPU, device=dev), randn_bf16((N_PER_GPU, N_PER_GPU), 1001))

        def two_plain():
            return layer2(layer(a))

        def two_chained():
            y, y_gs = layer(a, return_output_scale=True, next_layer=layer2)
            return layer2(y, x_global_scale=y_gs)

        for _ in range(3):
            two_plain(), two_chained()
        chain_steps = max(3, min(args.steps, 50))
        ms_two_plain = timed(two_plain, chain_steps, 6)
        ms_two_chained = timed(two_chained, chain_steps, 5)
        extra["two_layers_chained"] = {
            "what": "layer(a) -> layer2(.) at M=N=K=8192 each: every layer finds its activation's maximum itself, against "
                    "the first layer's GEMM epilogue handing the second its global scale",
            "ms_unchained": ms_two_plain, "ms_chained": ms_two_chained,
            "tflops_chained": 2 * 2.0 * M * N_PER_GPU * K / (ms_two_chained * 1e-3) / 1e12}
        del layer2
    del layer, gathered
    torch.cuda.empty_cache()
    if world > 1:
        extra["fp4_gather"] = {
            "what": "the same step with the output gathered as NVFP4 (packed nibbles + block scales written by the GEMM "
                    "epilogue into every rank's operand buffer) instead of bf16",
            "ms_per_step": ms_fp4_gather, "value": 2.0 * M * n_total * K / (ms_fp4_gather * 1e-3) / 1e12,
            "gather_bytes_out_per_rank": (world - 1) * M * N_PER_GPU * 9 // 16,
            "gather_gbs_per_rank": (world - 1) * M * N_PER_GPU * 0.5625 / (ms_fp4_gather * 1e-3) / 1e9}
    x_gu = randn_bf16((M, K), 2)
    cols = torch.randperm(K, generator=torch.Generator().manual_seed(2))[:K // 100].to(dev)
    x_gu[:, cols] *= 50
    n_gu_local = C4_GATE_UP_N // world
    if world > 1:
        gu = QuantLinear(K, C4_GATE_UP_N, parallel="column", fused_gather=fused, device=dev)
    else:
        gu = QuantLinear(K, C4_GATE_UP_N, device=dev)
    install_weight(gu, randn_bf16((n_gu_local, K), 2000 + rank, 0.02))
    gu.peer_wait_limit_ns = PEER_WAIT_NS
    gu.gather_output = True
    for _ in range(3):
        gu(x_gu)
    extra_steps = max(3, min(args.steps, 10))
    ms_gu = timed(lambda: gu(x_gu), extra_steps, 3)
    extra["c4_gate_up"] = {
        "layer": f"M{M} N{C4_GATE_UP_N} K{K}, column-parallel x{world}, output gathered on every rank",
        "ms": ms_gu, "tflops": 2.0 * M * C4_GATE_UP_N * K / (ms_gu * 1e-3) / 1e12,
        "gather_bytes_out_per_rank": (world - 1) * M * n_gu_local * 2,
        "gather_gbs_per_rank": (world - 1) * M * n_gu_local * 2 / (ms_gu * 1e-3) / 1e9}
    del gu, x_gu
    torch.cuda.empty_cache()

    k_dn_local = C4_DOWN_K // world
    x_dn = randn_bf16((M, k_dn_local), 3000 + rank)
    cols = torch.randperm(k_dn_local, generator=torch.Generator().manual_seed(3 + rank))[:max(1, k_dn_local // 100)].to(dev)
    x_dn[:, cols] *= 50
    if world > 1:
        dn = QuantLinear(C4_DOWN_K, N_PER_GPU, parallel="row", input_is_parallel=True, fused_reduce_scatter=fused, device=dev)
    else:
        dn = QuantLinear(C4_DOWN_K, N_PER_GPU, device=dev)
    install_weight(dn, randn_bf16((N_PER_GPU, k_dn_local), 4000 + rank, 0.02))
    dn.peer_wait_limit_ns = PEER_WAIT_NS
    for _ in range(3):
        y_dn = dn(x_dn)
    if world > 1:
        # (b) row-parallel: the fused reduce-scatter against NCCL's reduce_scatter of the fp32 partial products
        a_fp4, a_sf, alpha = dn._quantize_activation(x_dn)
        partial = dn._mm_f32(a_fp4, a_sf, alpha)
        ref = torch.empty((M // world, N_PER_GPU), dtype=torch.float32, device=dev)
        dist.reduce_scatter_tensor(ref, partial)
        row_ok, row_rel = gemm_tolerance(dn(x_dn), ref)
        parity["row_fused_max_rel" if fused else "row_nccl_max_rel"] = max_over_ranks(row_rel)
        row_ok = all_ranks(row_ok)
        parity["ok"] = bool(column_ok and slab_ok and row_ok and fp4_ok)
        parity["what"] = ("column: gathered [M, N_total] of this run's gather against the other gather (fused <-> NCCL) "
                          "of the same layer, torch.equal on every rank; own_slab: each rank's columns against the fp32 "
                          "product of the dequantized bytes the kernel consumed; row: Llama-3-70B down projection "
                          f"(M{M} N{N_PER_GPU} K{C4_DOWN_K}/{world}) against NCCL reduce_scatter_tensor of the fp32 "
                          "partial products; tolerance 1e-2 (max and per element, + 2^-8 rms)")
        del partial, ref, a_fp4, a_sf
    ms_dn = timed(lambda: dn(x_dn), extra_steps, 4 if world > 1 else 3)
    extra["c4_down"] = {
        "layer": f"M{M} N{N_PER_GPU} K{C4_DOWN_K}, row-parallel x{world}, " +
                 ("partial products reduce-scattered over the rows" if world > 1 else "single GPU"),
        "ms": ms_dn, "tflops": 2.0 * M * N_PER_GPU * C4_DOWN_K / (ms_dn * 1e-3) / 1e12,
        "reduce_bytes_out_per_rank": (world - 1) * (M // world) * N_PER_GPU * 4,
        "reduce_gbs_per_rank": (world - 1) * (M // world) * N_PER_GPU * 4 / (ms_dn * 1e-3) / 1e9}
    del dn, x_dn, y_dn

    status = nv.device_status()
    assert status == 0, f"a kernel gave up on a bounded wait (status {status:#x})"

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        if parity is not None and not parity["ok"]:
            raise SystemExit(3)
        return

    fp4_peak = 4.0 * peaks["bf16_tflops"]
    fp4_peak_sustained = 4.0 * peaks["bf16_tflops_sustained"]
    clocks, clocks_sustained = sampler.summary(), sustained_sampler.summary()
    mhz, mhz_s = clocks["sm_mhz"] or 0, clocks_sustained["sm_mhz"] or 0
    config = workload_config(world, args.gather)
    line = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp4_e2m1xue4m3_fp32acc", "data": "synthetic", "config": config,
        "kernels": {"gemm_ms": t_gemm, "gemm_tflops": gemm_tflops, "quant_ms": t_quant, "quant_gbs": quant_gbs,
                    "quant_frac_of_measured_hbm": quant_gbs / peaks["hbm_gbs"],
                    "quant_frac_of_nominal_8tbs": quant_gbs / NOMINAL_HBM_GBS,
                    "amax_ms": t_amax, "amax_gbs": amax_gbs,
                    "note": "each *_ms is the mean CUDA-event window around that one kernel in a pass of back-to-back "
                            "steps (three passes, one kernel timed per pass); a window holds the kernel plus its launch "
                            "gap and drain.  Inside a step the three kernels OVERLAP: the launches are chained with "
                            "programmatic dependent launch (the quantizer loads its tiles under the tail of the amax "
                            "sweep; the GEMM sets up and fetches its first weight stages under the tail of the "
                            "quantizer), so amax_ms + quant_ms + gemm_ms exceeds ms_per_step"},
        "sustained": {"ms_per_step": ms_sustained, "value": flops_step / (ms_sustained * 1e-3) / 1e12,
                      "steps": sustained_steps, "gemm_ms": t_gemm_sustained, "gemm_tflops": gemm_tflops_sustained,
                      "gemm_frac_of_4x_sustained_bf16": gemm_tflops_sustained / fp4_peak_sustained,
                      "gemm_frac_of_nominal_9pflops": gemm_tflops_sustained / NOMINAL_FP4_TFLOPS,
                      "sm_mhz_median": clocks_sustained["sm_mhz"], "reasons": clocks_sustained["reasons"],
                      "gemm_ms_x_mhz": t_gemm_sustained * mhz_s, "burst_gemm_ms_x_mhz": t_gemm * mhz,
                      "note": "the step, and separately the step with an event pair around its GEMM, each repeated for "
                              "at least 1.2 s; burst figures (value, kernels, roofline) come from --steps steps"},
        "roofline": {"bound": "tensor", "achieved": gemm_tflops, "peak": fp4_peak, "unit": "TFLOP/s",
                     "frac": gemm_tflops / fp4_peak, "traffic": GEMM_DRAM_BYTES_PER_LAUNCH,
                     "traffic_unit": "bytes per launch, dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture "
                                     "of this launch (profiles/fp4_gemm_pair_kernel_8192.txt); algorithmic bytes: "
                                     f"{GEMM_ALGORITHMIC_BYTES / 1e6:.1f} MB",
                     "kernel": "fp4_gemm_pair_kernel",
                     "peak_basis": f"burst: 4 x {peaks['source']} dense bf16 burst ({peaks['bf16_tflops']} TFLOP/s), the "
                                   "kernel timed over --steps steps; sustained.gemm_frac_of_4x_sustained_bf16 uses 4 x "
                                   f"the sustained bf16 figure ({peaks['bf16_tflops_sustained']} TFLOP/s); no FP4 peak is "
                                   "measured on this pool",
                     "frac_of_nominal_9pflops": gemm_tflops / NOMINAL_FP4_TFLOPS,
                     "algorithmic_flops_per_launch": 2.0 * M * N_PER_GPU * K},
        "e2e": {"value": e2e_value, "unit": "TFLOP/s", "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": world * a_host.numel() * 2, "d2h_bytes_per_step": world * out_host.numel() * 2,
                "bytes_note": "totals over all ranks: the activation crosses PCIe once per step (each rank copies 1/N of "
                              "its rows, the ranks all-gather the pieces over NVLink); every rank copies its own column "
                              "slab of the result out",
                "how": "nvfp_kernel_b200.HostPipeline(depth=2): pinned host input copied in, layer, result copied out to "
                       "pinned host memory, every step; consecutive steps overlap on three streams",
                "serial_ms_per_step": ms_e2e_serial,
                "serial_value": flops_step / (ms_e2e_serial * 1e-3) / 1e12},
        "extra": extra,
        "gpu_launches": own_launches[0],
        "launches_per_step": launches_per_step,
        "clocks": clocks,
    }
    if parity is not None:
        line["parity"] = parity
        line["nvlink"] = nvlink
    if world == 1 and not args.no_cpu_baseline:
        tflops, cores, sample, _, _ = run_cpu_baseline(20.0, 3, 1)
        line["cpu_baseline"] = {"value": tflops, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    if parity is not None and not parity["ok"]:
        raise SystemExit(3)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--profile-mode", action="store_true",
                    help="run only the warm-up and the burst region (for ncu captures of the step's kernels)")
    ap.add_argument("--gather", default="fused", choices=["fused", "nccl", "fused-fp4"],
                    help="N>1 only: how the column-parallel outputs are gathered (fused-fp4: as NVFP4, for a next "
                         "quantized layer)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        main_reference(args, rank)
        return
    if world != args.gpus:
        if args.gpus == 1 and world == 1:
            pass
        else:
            raise SystemExit(f"--gpus {args.gpus} needs a launch with WORLD_SIZE={args.gpus} "
                             f"(python -m torch.distributed.run --nproc-per-node {args.gpus} ...); got {world}")
    main_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
