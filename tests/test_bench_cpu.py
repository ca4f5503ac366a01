"""bench.py's own checking code, on CPU: the dequantizer and the tolerance rule it uses for the N > 1 parity block
against the oracle, and the `config` both arms print."""
import importlib.util
import os

import numpy as np
import torch

from inputs import make_input
from oracle import nvfp_oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_dequantizer_of_the_parity_block_matches_the_oracle():
    bench = _bench()
    x = make_input("normal", (130, 192), torch.bfloat16, 5)
    gs = O.global_scale_from_amax(x.float().abs().max().item())
    fp4, sf, _ = O.nvfp4_quantize_kernel(x, gs)
    got = bench.dequantize_fp32(torch.from_numpy(fp4), torch.from_numpy(sf))
    want = O.dequantize(fp4, sf, 1.0, block=16, scale_format="e4m3")          # value * block scale, no global scale
    assert got.dtype == torch.float32 and np.array_equal(got.double().numpy(), want)


def test_tolerance_rule_of_the_parity_block():
    bench = _bench()
    g = torch.Generator().manual_seed(0)
    ref = torch.randn((64, 64), generator=g)
    ok, rel = bench.gemm_tolerance(ref.to(torch.bfloat16), ref)               # bf16 rounding: inside
    assert ok and rel < 2.0 ** -8
    bad = ref.clone()
    bad[3, 5] += 0.05 * ref.abs().max()                                       # one element 5 % of max off: outside
    assert not bench.gemm_tolerance(bad, ref)[0]
    nan = ref.clone()
    nan[0, 0] = float("nan")
    assert not bench.gemm_tolerance(nan, ref)[0]
    small = ref.clone()
    small += 2.0 ** -10 * ref.pow(2).mean().sqrt()                            # a shift far below 2^-8 rms: inside
    assert bench.gemm_tolerance(small, ref)[0]


def test_both_arms_describe_the_same_workload():
    bench = _bench()
    for world in (1, 2, 8):
        ours = bench.workload_config(world, "fused")
        assert ours["workload"] == f"nvfp4_quant_linear_M8192_N8192x{world}_K8192"
        assert bench.workload_config(world, "fused") == ours
    assert "NVFP4" in bench.workload_config(4, "fused-fp4")["parallelism"]
    assert bench.workload_config(1, "nccl")["parallelism"] == "single GPU"
