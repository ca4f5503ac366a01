"""Generates tests/golden/ref_torch_path.npz by RUNNING the reference's own torch
pseudo-quant path (nvfp/pseudo_quant.py of the reference checkout) on CPU.

Usage (needs the reference checkout; run once, commit the .npz):
    python tests/golden/make_ref_torch_golden.py /path/to/reference

Three shims make the reference module importable without a GPU; none of them
changes its arithmetic:
  1. an empty ``expecttest`` module, which ``torch.testing._internal`` imports;
  2. ``torch.tensor(..., device="cuda")`` at import time is redirected to the CPU
     (the e2m1 look-up table, nvfp/pseudo_quant.py:103-116);
  3. ``reciprocal_approximate_ftz_tensor`` (a CUDA-only op) is replaced by the
     correctly rounded fp32 reciprocal 1/x.
The fixture therefore pins the oracle's ``nvfp4_quantize_torch_path`` with
``rcp_true``, its swizzle, its dequantize and its e2m1/e4m3 codecs.
"""
import hashlib
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
from inputs import DISTRIBUTIONS, make_input, c1_inputs  # noqa: E402


def import_reference(ref_root: str):
    stub = types.ModuleType("expecttest")
    stub.TestCase = object
    sys.modules.setdefault("expecttest", stub)
    sys.path.insert(0, ref_root)
    real_tensor = torch.tensor

    def cpu_tensor(*a, **kw):
        if kw.get("device") == "cuda":
            kw["device"] = "cpu"
        return real_tensor(*a, **kw)

    torch.tensor = cpu_tensor
    try:
        import nvfp.pseudo_quant as pq
    finally:
        torch.tensor = real_tensor
    pq.reciprocal_approximate_ftz_tensor = lambda t: (1.0 / t.double()).float()
    return pq


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def main():
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("NVFP_REFERENCE_ROOT")
    if not ref_root:
        raise SystemExit("usage: make_ref_torch_golden.py /path/to/reference  (or set NVFP_REFERENCE_ROOT)")
    pq = import_reference(ref_root)
    out = {}

    # e2m1 codec: every interesting fp32 input through the reference's to_fp4
    probe = torch.tensor([0.0, -0.0, 0.1, 0.25, 0.2500001, 0.5, 0.75, 0.7499999, 1.0, 1.25, 1.2500001,
                          1.5, 1.75, 2.0, 2.5, 2.5000002, 3.0, 3.5, 4.0, 5.0, 5.0000005, 6.0, 7.0, 100.0,
                          -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0, -6.0, -1e-30, 1e-30, -0.1, 0.3],
                         dtype=torch.float32)
    out["e2m1_probe_in"] = probe.numpy()
    out["e2m1_probe_packed"] = pq.to_fp4(probe.reshape(1, -1)).view(torch.uint8).numpy()

    # small cases: all 7 distributions, fp16 and bf16, two shapes
    for dist in DISTRIBUTIONS:
        for shape in ((128, 128), (129, 80)):
            for dt_name, dt in (("bf16", torch.bfloat16), ("fp16", torch.float16)):
                x = make_input(dist, shape, dt, seed=11)
                fp4, sf_swz, gs = pq.quantize_linear_weight_to_nvfp4(x)
                _, sf_lin = pq.pytorch_nvfp4_quantize(x, gs)
                # the reference's dequantize slices the scale tensor with K instead of K/16
                # (nvfp/pseudo_quant.py:175) and so only works when K/16 is a multiple of 4
                deq = pq.dequantize_to_dtype(fp4, sf_swz, gs, 16) if (shape[1] // 16) % 4 == 0 else None
                key = f"{dist}_{shape[0]}x{shape[1]}_{dt_name}"
                out[key + "_x"] = x.view(torch.int16).numpy()
                out[key + "_gs"] = gs.numpy().reshape(1)
                out[key + "_fp4"] = fp4.view(torch.uint8).numpy()
                out[key + "_sf_lin"] = sf_lin.view(torch.uint8).numpy()
                # swizzled tensor: padding is uninitialised in the reference; keep valid part only
                sf_valid = pq.swizzled_to_linear_128_4(sf_swz.view(torch.uint8), shape[0], shape[1] // 16)
                out[key + "_sf_unswz"] = sf_valid.numpy()
                if deq is not None:
                    out[key + "_deq"] = deq.numpy()

    # swizzle permutation on an index ramp (exactly defined everywhere: no padding)
    ramp = torch.arange(256 * 8, dtype=torch.int32).reshape(256, 8)
    out["swizzle_ramp"] = pq.linear_to_swizzled_128_4(ramp).numpy()

    # BASELINE config 1: A [1024,1024] ~N(0,1) bf16, W ~N(0,1/sqrt(K)) bf16, seed 0
    a, w = c1_inputs()
    a_fp4, a_sf, a_gs = pq.quantize_linear_weight_to_nvfp4(a)
    w_fp4, w_sf, w_gs = pq.quantize_linear_weight_to_nvfp4(w)
    a_dq = pq.dequantize_to_dtype(a_fp4, a_sf, a_gs, 16)
    w_dq = pq.dequantize_to_dtype(w_fp4, w_sf, w_gs, 16)
    y = (a_dq @ w_dq.T)
    out["c1_a_sha"] = np.frombuffer(bytes.fromhex(sha(a.view(torch.int16).numpy())), dtype=np.uint8)
    out["c1_w_sha"] = np.frombuffer(bytes.fromhex(sha(w.view(torch.int16).numpy())), dtype=np.uint8)
    out["c1_a_gs"] = a_gs.numpy().reshape(1)
    out["c1_w_gs"] = w_gs.numpy().reshape(1)
    out["c1_a_fp4_sha"] = np.frombuffer(bytes.fromhex(sha(a_fp4.view(torch.uint8).numpy())), dtype=np.uint8)
    out["c1_w_fp4_sha"] = np.frombuffer(bytes.fromhex(sha(w_fp4.view(torch.uint8).numpy())), dtype=np.uint8)
    out["c1_a_sf_sha"] = np.frombuffer(bytes.fromhex(sha(a_sf.view(torch.uint8).numpy())), dtype=np.uint8)
    out["c1_w_sf_sha"] = np.frombuffer(bytes.fromhex(sha(w_sf.view(torch.uint8).numpy())), dtype=np.uint8)
    out["c1_a_fp4_head"] = a_fp4.view(torch.uint8).numpy()[:64]
    out["c1_y_corner"] = y[:64, :64].numpy()          # float64, unrounded
    out["c1_y_rows"] = y[::97].numpy()                # every 97th row, float64

    path = os.path.join(HERE, "ref_torch_path.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    main()
