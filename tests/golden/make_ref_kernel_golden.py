"""Generates ref_kernel_sm100.npz and ref_kernel_ue8m0_sm100.npz by RUNNING the reference's own CUDA quantizer
(kernel/nvfp4_quant_kernels.cu of the reference, built for sm_100a by
oracle/build_oracle.py into oracle/_ref/) on a B200.

    python tests/golden/make_ref_kernel_golden.py OUT_DIR

For every case it stores the kernel's packed nibbles, its scale bytes (valid region only:
the reference leaves padding uninitialised), the global scale, and the results of the
reference's reciprocal_approximate_ftz_tensor for every value the quantizer can feed to
rcp.approx.ftz with that global scale, so that the CPU oracle can replay the hardware
reciprocal exactly.  Inputs are the seeded tensors of tests/golden/inputs.py (seed 11): the reference's seven
distributions, `zeros_mixed` and `specials` (infinities, NaNs, -0, denormals; global scale 672 for that one).
"""
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path[:0] = [HERE, ROOT]
from inputs import DISTRIBUTIONS, make_input, mx_duplicated_halves  # noqa: E402
from oracle import nvfp_oracle as O  # noqa: E402

CASE_DISTS = DISTRIBUTIONS + ("zeros_mixed", "specials")
CASE_SHAPES = ((128, 128), (129, 80))


def load_ref():
    d = os.path.join(ROOT, "oracle", "_ref")
    name = [f for f in os.listdir(d) if f.startswith("ref_scaled_fp4_ops") and f.endswith(".so")][0]
    spec = importlib.util.spec_from_file_location("ref_scaled_fp4_ops", os.path.join(d, name))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def ref_quant(ref, x, gs):
    m, n = x.shape
    out = torch.empty((m, n // 2), dtype=torch.uint8, device="cuda")
    rm, rn = (m + 127) // 128 * 128, (n // 16 + 3) // 4 * 4
    sf = torch.zeros((rm, rn // 4), dtype=torch.int32, device="cuda")
    ref.scaled_fp4_quant_sm1xxa(out, x, sf, gs)
    return out, sf.view(torch.uint8).reshape(rm, rn)


def ref_rcp(ref, t):
    y = torch.zeros_like(t)
    ref.reciprocal_approximate_ftz_tensor(t, y)
    return y


def main():
    out_dir = sys.argv[1] if len(sys.argv) > 1 else "."
    ref = load_ref()
    out = {}
    for dist in CASE_DISTS:
        for shape in CASE_SHAPES:
            for dt_name, dt in (("bf16", torch.bfloat16), ("fp16", torch.float16)):
                x = make_input(dist, shape, dt, seed=11)
                finite = x.float()[torch.isfinite(x.float())]
                amax = finite.abs().max() if dist != "specials" else torch.tensor(4.0)
                gs = (torch.tensor(448.0 * 6.0) / (amax if amax > 0 else torch.tensor(1.0))).to(torch.float32)
                xg, gsg = x.cuda(), gs.reshape(1).cuda()
                fp4, sf = ref_quant(ref, xg, gsg)
                first = torch.tensor([6.0, gs.item()], dtype=torch.float32, device="cuda")
                r1 = ref_rcp(ref, first)
                second = torch.from_numpy(O.rcp_second_pass_inputs(r1[1].item())).cuda()
                r2 = ref_rcp(ref, second)
                key = f"{dist}_{shape[0]}x{shape[1]}_{dt_name}"
                out[key + "_gs"] = gs.numpy().reshape(1)
                out[key + "_fp4"] = fp4.cpu().numpy()
                out[key + "_sf"] = O.unswizzle_128x4(sf.cpu().numpy(), shape[0], shape[1] // 16)
                out[key + "_rcp_in"] = torch.cat([first, second]).cpu().numpy()
                out[key + "_rcp_out"] = torch.cat([r1, r2]).cpu().numpy()
                if dist in ("zeros_mixed", "specials"):
                    out[key + "_x"] = x.view(torch.int16).numpy()
    path = os.path.join(out_dir, "ref_kernel_sm100.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")

    # The reference's e8m0 branch (cvt_warp_fp16_to_fp4<Type, true>, kernel/nvfp4_utils.cuh:196-202; 16-element blocks,
    # no global scale), run through its own launcher template: pins MXFP4's `floor` scale rounding.  Inputs: every
    # 32-block two copies of one 16-element half (inputs.mx_duplicated_halves, seed 17).
    if hasattr(ref, "scaled_fp4_quant_ue8m0"):
        mx = {}
        for dist in CASE_DISTS + ("student_t3",):
            for shape in ((128, 128), (129, 96)):
                for dt_name, dt in (("bf16", torch.bfloat16), ("fp16", torch.float16)):
                    x = mx_duplicated_halves(dist, shape, dt, seed=17).cuda()
                    m, n = shape
                    fp4 = torch.empty((m, n // 2), dtype=torch.uint8, device="cuda")
                    rm, rn = (m + 127) // 128 * 128, (n // 16 + 3) // 4 * 4
                    sf = torch.zeros((rm, rn // 4), dtype=torch.int32, device="cuda")
                    ref.scaled_fp4_quant_ue8m0(fp4, x, sf)
                    key = f"{dist}_{m}x{n}_{dt_name}"
                    mx[key + "_fp4"] = fp4.cpu().numpy()
                    mx[key + "_sf16"] = O.unswizzle_128x4(sf.view(torch.uint8).reshape(rm, rn).cpu().numpy(), m, n // 16)
        path = os.path.join(out_dir, "ref_kernel_ue8m0_sm100.npz")
        np.savez_compressed(path, **mx)
        print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
