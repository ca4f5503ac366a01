#!/usr/bin/env python
"""Benchmark of the NVFP4 hot path: activation amax + quantize -> block-scaled FP4 GEMM.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one forward of QuantLinear(mode="real") on M=N=K=8192 (per GPU): global scale
of the bf16 activation, NVFP4 quantize, alpha, FP4 GEMM with bf16 output (the flow of the
reference's speed_test.py:36-50; the weight is quantized once, outside the timed region).
With N>1 the layer is column-parallel: every rank holds 8192 output columns (weak scaling)
and the step ends with the all-gather of the bf16 outputs.

Prints ONE JSON line (rank 0).  `value` = 2*M*N_total*K / step time in TFLOP/s with the
activation resident in HBM; `e2e` = the same through the public Python API with the
activation in pinned host memory and the output copied back; `roofline` describes the GEMM
kernel (timed alone inside the run with CUDA events); `cpu_baseline` is the CPU port of the
reference's torch pseudo-quant path on a bounded sample.

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
METRIC = "nvfp4_gemm_tflops_m8192_n8192_k8192"
NOMINAL_FP4_TFLOPS = 9000.0
NOMINAL_HBM_GBS = 8000.0
# DRAM bytes the GEMM launch of this workload moved under ncu (96.4 MB read + 108.1 MB written: both operands and
# their scales read once; of the 134 MB of output, 108 MB reached DRAM before the kernel ended, the rest sat in L2).
GEMM_DRAM_BYTES_PER_LAUNCH = 204.5e6
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
    """Returns (TFLOP/s, cores, sample description, ms per step)."""
    step = cpu_reference_step_factory()
    t_probe = step(64)
    rows = int(max(16, min(1024, (budget_s / max(1, steps + warmup)) / (t_probe / 64))) // 16 * 16)
    for _ in range(warmup):
        step(rows)
    times = [step(rows) for _ in range(steps)]
    t = sum(times) / len(times)
    tflops = 2.0 * rows * N_PER_GPU * K / t / 1e12
    sample = (f"{rows} of {M} activation rows per step (quantize + dequantize + float64 matmul against the full "
              f"[{N_PER_GPU},{K}] dequantized weight; weight side prepared once, untimed), mean of {steps} steps")
    return tflops, torch.get_num_threads(), sample, t * 1e3


def main_reference(args, rank: int):
    if rank != 0:
        return
    tflops, cores, sample, ms = run_cpu_baseline(120.0, args.steps, args.warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": tflops, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": {"workload": f"nvfp4_quant_linear_M{M}_N{N_PER_GPU}_K{K}", "note":
                   "CPU port of the reference's torch pseudo-quant path (the reference's CUDA GEMM is sm_120a-only "
                   "and cannot run on B200); bounded row sample per step"},
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------- GPU arm ---
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

    # synthetic data: activations ~N(0,1) (same on every rank), weights ~N(0,1) as in the
    # reference's speed_test.py:74-75; each rank draws only its own 8192 output columns
    g = torch.Generator(device=dev).manual_seed(0)
    a = torch.randn((M, K), generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
    gw = torch.Generator(device=dev).manual_seed(1000 + rank)
    w_local = torch.randn((N_PER_GPU, K), generator=gw, device=dev, dtype=torch.float32).to(torch.bfloat16)

    if world > 1:
        # this rank's column slab of a column-parallel layer; the gather is fused into the GEMM epilogue
        # (peer stores over NVLink) unless --gather nccl asks for the all-gather collective
        layer = QuantLinear(K, n_total, parallel="column", fused_gather=(args.gather == "fused"), device=dev)
    else:
        layer = QuantLinear(K, N_PER_GPU, device=dev)
    if world > 1:
        # one global weight scale for the whole [n_total, K] weight, as a 1-GPU layer would use
        amax = w_local.float().abs().max().reshape(1)
        dist.all_reduce(amax, op=dist.ReduceOp.MAX)
        gs_w = (2688.0 / amax).to(torch.float32)
        w_fp4, w_sf = nv.scaled_fp4_quant(w_local, gs_w)
        layer.weight_fp4, layer.weight_sf = w_fp4, w_sf.view(torch.uint8)
        layer.weight_global_scale.copy_(gs_w)
    else:
        layer.load_weight(w_local)
    del w_local
    gathered = torch.empty((world * M, N_PER_GPU), dtype=torch.bfloat16, device=dev) if world > 1 else None
    layer.gather_output = args.gather == "fused"

    def step(x):
        y = layer(x)                     # fused gather: already the full [M, n_total] matrix
        if world > 1 and args.gather == "nccl":
            dist.all_gather_into_tensor(gathered, y)     # layout [world, M, N/world]
            return gathered
        return y

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

    sampler = ClockSampler(local_rank)
    launches_per_step = 3 if world == 1 or args.gather == "fused" else 4   # amax(+scales), quantize, gemm (+ all-gather)
    own_kernels_per_step = 3

    for _ in range(max(3, args.warmup)):
        step(a)
    barrier()

    # ---- region 1: whole hot path, activation resident in HBM ------------------------
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with sampler:
        barrier()
        e0.record()
        for _ in range(args.steps):
            step(a)
        e1.record()
        barrier()
    ms_step = max_over_ranks(e0.elapsed_time(e1) / args.steps)
    flops_step = 2.0 * M * n_total * K
    value = flops_step / (ms_step * 1e-3) / 1e12

    # ---- region 2: the same steps with an event pair around ONE of the kernels (kernel breakdown) ---
    # calls the same ops QuantLinear.forward makes, one by one; three passes, each timing one kernel of every step
    # (a pair of events around every kernel of a step would put six event records, and their gaps, into each step)
    ks = min(args.steps, 200)
    w_sf = layer.weight_sf.view(torch.float8_e4m3fn)

    def timed_pass(which: int) -> float:
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
        return statistics.mean(e0.elapsed_time(e1) for e0, e1 in ev)

    with sampler:
        t_amax, t_quant, t_gemm = timed_pass(0), timed_pass(1), timed_pass(2)
    gemm_tflops = 2.0 * M * N_PER_GPU * K / (t_gemm * 1e-3) / 1e12
    quant_bytes = M * K * 2.5625
    quant_gbs = quant_bytes / (t_quant * 1e-3) / 1e9
    amax_gbs = M * K * 2.0 / (t_amax * 1e-3) / 1e9

    # ---- region 3: end to end through the public API with host buffers -----------------
    a_host = a.cpu().pin_memory()
    # Every rank ends a step holding the whole gathered [M, n_total] result; the host needs it once, so each rank
    # copies out its own [M, N_PER_GPU] column slab (all ranks together: the whole result, every step).
    out_host = torch.empty((M * N_PER_GPU,), dtype=torch.bfloat16).pin_memory()
    a_dev = torch.empty_like(a)
    e2e_steps = max(3, min(args.steps, 20))

    def step_for_host(x):
        y = step(x)
        if world == 1:
            return y
        if args.gather == "nccl":
            return y.view(world, M, N_PER_GPU)[rank]            # all_gather_into_tensor's layout: [world, M, N/world]
        return y[:, rank * N_PER_GPU:(rank + 1) * N_PER_GPU]     # this rank's columns of the gathered matrix

    def e2e_step():
        a_dev.copy_(a_host, non_blocking=True)
        y = step_for_host(a_dev)
        out_host.copy_(y.reshape(-1), non_blocking=True)

    for _ in range(2):
        e2e_step()
    with sampler:
        barrier()
        e0.record()
        for _ in range(e2e_steps):
            e2e_step()
        e1.record()
        barrier()
    ms_e2e_serial = max_over_ranks(e0.elapsed_time(e1) / e2e_steps)

    # the same calls through HostPipeline: the copy-in of step i+1, the kernels of step i and the copy-out of step
    # i-1 run at the same time (PCIe is full duplex); every step still copies its own input in and its result out
    pipe = nv.HostPipeline(step_for_host, depth=2, device=dev, reuses_output=world > 1)
    out_hosts = [out_host, torch.empty_like(out_host).pin_memory()]
    for i in range(3):
        pipe.submit(a_host, out_hosts[i % 2])
    pipe.synchronize()
    with sampler:
        barrier()
        e0.record(pipe.copy_in)
        for i in range(e2e_steps):
            pipe.submit(a_host, out_hosts[i % 2])
        e1.record(pipe.copy_out)
        pipe.synchronize()
        barrier()
    ms_e2e = max_over_ranks(e0.elapsed_time(e1) / e2e_steps)
    e2e_value = flops_step / (ms_e2e * 1e-3) / 1e12
    status = nv.device_status()
    assert status == 0, f"a kernel gave up on a bounded wait (status {status:#x})"

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    fp4_peak = 4.0 * peaks["bf16_tflops"]
    line = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(3, args.warmup), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp4_e2m1xue4m3_fp32acc", "data": "synthetic",
        "config": {"workload": f"nvfp4_quant_linear_M{M}_N{N_PER_GPU}x{world}_K{K}",
                   "step": "amax -> global scale and alpha (one kernel), NVFP4 quantize of the bf16 activation, FP4 GEMM, bf16 out"
                           + (", all-gather of outputs (column-parallel)" if world > 1 else ""),
                   "parallelism": (f"column-parallel x{world}, gather " + ("fused into the GEMM epilogue (peer stores)"
                                   if args.gather == "fused" else "by NCCL all-gather")) if world > 1 else "single GPU",
                   "l2": "no flush: bf16 activation (134 MB) + output (134 MB) per step exceed the 126 MB L2"},
        "kernels": {"gemm_ms": t_gemm, "gemm_tflops": gemm_tflops, "quant_ms": t_quant, "quant_gbs": quant_gbs,
                    "quant_frac_of_measured_hbm": quant_gbs / peaks["hbm_gbs"],
                    "quant_frac_of_nominal_8tbs": quant_gbs / NOMINAL_HBM_GBS,
                    "amax_ms": t_amax, "amax_gbs": amax_gbs},
        "roofline": {"bound": "tensor", "achieved": gemm_tflops, "peak": fp4_peak, "unit": "TFLOP/s",
                     "frac": gemm_tflops / fp4_peak, "traffic": GEMM_DRAM_BYTES_PER_LAUNCH,
                     "traffic_unit": "bytes per launch, dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture "
                                     "of this launch (profiles/fp4_gemm_pair_kernel_8192.txt); algorithmic bytes: "
                                     f"{GEMM_ALGORITHMIC_BYTES / 1e6:.1f} MB",
                     "kernel": "fp4_gemm_pair_kernel",
                     "peak_basis": f"4 x {peaks['source']} dense bf16 burst ({peaks['bf16_tflops']} TFLOP/s); "
                                   "no FP4 peak is measured on this pool",
                     "frac_of_nominal_9pflops": gemm_tflops / NOMINAL_FP4_TFLOPS,
                     "algorithmic_flops_per_launch": 2.0 * M * N_PER_GPU * K},
        "e2e": {"value": e2e_value, "unit": "TFLOP/s", "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": world * a_host.numel() * 2, "d2h_bytes_per_step": world * out_host.numel() * 2,
                "bytes_note": "totals over all ranks: every rank copies the (replicated) activation in and its own "
                              "column slab of the result out",
                "how": "nvfp_kernel_b200.HostPipeline(depth=2): pinned host input copied in, layer, result copied out to "
                       "pinned host memory, every step; consecutive steps overlap on three streams",
                "serial_ms_per_step": ms_e2e_serial,
                "serial_value": flops_step / (ms_e2e_serial * 1e-3) / 1e12},
        "gpu_launches": own_kernels_per_step * (args.steps + 3 * ks + 2 * e2e_steps),
        "launches_per_step": launches_per_step,
        "clocks": sampler.summary(),
    }
    if world == 1 and not args.no_cpu_baseline:
        tflops, cores, sample, _ = run_cpu_baseline(20.0, 3, 1)
        line["cpu_baseline"] = {"value": tflops, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--gather", default="fused", choices=["fused", "nccl"],
                    help="N>1 only: how the column-parallel outputs are gathered")
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
