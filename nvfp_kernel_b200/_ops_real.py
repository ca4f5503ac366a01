"""Wrappers over the `scaled_fp4_ops` extension: input checks and output allocation.

Mirror of the reference's nvfp/_ops_real.py:25-98 (same asserts, shapes and dtypes of
the results) plus the MXFP4 and helper entry points.  The extension is looked up by
module name like the reference does (nvfp/_ops_real.py:8), then in this package's own
directory where the in-tree build puts it.
"""
from __future__ import annotations

import importlib
import importlib.util
import os
import sys

import torch

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))


def _load_scaled_fp4_ops(required_symbols: tuple[str, ...]):
    module = sys.modules.get("scaled_fp4_ops")
    if module is None:
        try:
            module = importlib.import_module("scaled_fp4_ops")
        except ImportError:
            module = None
            for name in sorted(os.listdir(_PKG_DIR)):
                if name.startswith("scaled_fp4_ops") and name.endswith(".so"):
                    spec = importlib.util.spec_from_file_location("scaled_fp4_ops", os.path.join(_PKG_DIR, name))
                    module = importlib.util.module_from_spec(spec)
                    spec.loader.exec_module(module)
                    sys.modules["scaled_fp4_ops"] = module
                    break
            if module is None:
                raise RuntimeError(
                    "scaled_fp4_ops extension is not available. "
                    "Build it with `python -m nvfp_kernel_b200.build` (sm_100a; no fallback exists)."
                ) from None
    missing = [name for name in required_symbols if not hasattr(module, name)]
    if missing:
        raise RuntimeError(
            "scaled_fp4_ops is missing required real-kernel symbols: "
            f"{', '.join(missing)}. Rebuild with `python -m nvfp_kernel_b200.build --force`.")
    return module


def _round_up(x: int, y: int) -> int:
    return (x + y - 1) // y * y


def _quant_common(input: torch.Tensor, block_size: int):
    assert input.is_cuda, "input must be a CUDA tensor"
    assert input.ndim >= 1, f"input.ndim needs to be >= 1, but got {input.ndim}."
    other_dims = 1 if input.ndim == 1 else -1
    input = input.reshape(other_dims, input.shape[-1])
    m, n = input.shape
    assert n % block_size == 0, f"last dim has to be multiple of {block_size}, but got {n}."
    assert input.dtype in (torch.float16, torch.bfloat16), \
        f"input.dtype needs to be fp16 or bf16 but got {input.dtype}."
    if input.stride(-1) != 1 or (m > 1 and input.stride(0) % 8 != 0) or input.data_ptr() % 16 != 0:
        input = input.contiguous()
    output = torch.empty((m, n // 2), device=input.device, dtype=torch.uint8)
    rounded_m = _round_up(m, 128)
    rounded_n = _round_up(n // block_size, 4)
    output_scale = torch.empty((rounded_m, rounded_n // 4), device=input.device, dtype=torch.int32)
    return input, output, output_scale


def scaled_fp4_quant(input: torch.Tensor, input_global_scale: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """bf16/fp16 [..., n] -> (uint8 [m, n/2], float8_e4m3fn [round_up(m,128), round_up(n/16,4)])."""
    assert input_global_scale.is_cuda, "input_global_scale must be a CUDA tensor"
    assert input_global_scale.dtype == torch.float, \
        f"input_global_scale.dtype needs to be fp32 but got {input_global_scale.dtype}."
    input, output, output_scale = _quant_common(input, 16)
    ext = _load_scaled_fp4_ops(("scaled_fp4_quant_sm1xxa",))
    ext.scaled_fp4_quant_sm1xxa(output, input, output_scale, input_global_scale)
    return output, output_scale.view(torch.float8_e4m3fn)


def scaled_mxfp4_quant(input: torch.Tensor, rounding: str = "rceil") -> tuple[torch.Tensor, torch.Tensor]:
    """bf16/fp16 [..., n] -> (uint8 [m, n/2], float8_e8m0fnu [round_up(m,128), round_up(n/32,4)])."""
    assert rounding in ("rceil", "floor"), f"rounding must be 'rceil' or 'floor', got {rounding!r}"
    input, output, output_scale = _quant_common(input, 32)
    ext = _load_scaled_fp4_ops(("scaled_mxfp4_quant",))
    ext.scaled_mxfp4_quant(output, input, output_scale, 0 if rounding == "rceil" else 1)
    return output, output_scale.view(torch.float8_e8m0fnu)


def _mm_asserts(a, b, block_scale_a, block_scale_b, alpha, out_dtype, sf_dtype):
    assert a.is_cuda, "a must be a CUDA tensor"
    assert b.is_cuda, "b must be a CUDA tensor"
    assert block_scale_a.is_cuda, "block_scale_a must be a CUDA tensor"
    assert block_scale_b.is_cuda, "block_scale_b must be a CUDA tensor"
    assert a.ndim == 2 and b.ndim == 2
    assert a.dtype in (torch.uint8,), f"a.dtype needs to be uint8 but got {a.dtype}"
    assert b.dtype in (torch.uint8,), f"b.dtype needs to be uint8 but got {b.dtype}"
    assert block_scale_a.dtype in (sf_dtype,), f"block_scale_a.dtype needs to be {sf_dtype} but got {block_scale_a.dtype}"
    assert block_scale_b.dtype in (sf_dtype,), f"block_scale_b.dtype needs to be {sf_dtype} but got {block_scale_b.dtype}"
    if alpha is not None:
        assert alpha.is_cuda, "alpha must be a CUDA tensor"
        assert alpha.dtype == torch.float, f"alpha.dtype needs to be fp32 but got {alpha.dtype}"
    assert out_dtype in (torch.float16, torch.bfloat16), f"out_dtype needs to be fp16 or bf16 but got {out_dtype}"


def _check_bias(bias, n, out_dtype):
    assert bias.is_cuda, "bias must be a CUDA tensor"
    assert bias.ndim == 1 and bias.shape[0] == n, f"bias must have shape ({n},) but got {tuple(bias.shape)}"
    assert bias.dtype == out_dtype, f"bias.dtype needs to be {out_dtype} but got {bias.dtype}"
    return bias.contiguous()


def cutlass_scaled_fp4_mm(a, b, block_scale_a, block_scale_b, alpha, out_dtype, bias=None) -> torch.Tensor:
    """out[m,n] = alpha * (a*sfa) @ (b*sfb)^T (+ bias[n], added in the epilogue before the single rounding).
    The name is the reference's; the kernel is the hand-written tcgen05 one (no CUTLASS); `bias` is an addition."""
    assert alpha is not None, "alpha must be a CUDA tensor"
    _mm_asserts(a, b, block_scale_a, block_scale_b, alpha, out_dtype, torch.float8_e4m3fn)
    m, n = a.shape[0], b.shape[0]
    out = torch.empty((m, n), dtype=out_dtype, device=a.device)
    if bias is not None:
        ext = _load_scaled_fp4_ops(("scaled_fp4_mm_bias",))
        ext.scaled_fp4_mm_bias(out, a, b, block_scale_a, block_scale_b, alpha, _check_bias(bias, n, out_dtype), False)
        return out
    ext = _load_scaled_fp4_ops(("cutlass_scaled_fp4_mm",))
    ext.cutlass_scaled_fp4_mm(out, a, b, block_scale_a, block_scale_b, alpha)
    return out


def scaled_fp4_mm_fp4out(a, b, block_scale_a, block_scale_b, alpha, out_global_scale, value_dtype=torch.bfloat16,
                         bias=None) -> tuple[torch.Tensor, torch.Tensor]:
    """scaled_fp4_quant(cutlass_scaled_fp4_mm(a, b, ..., value_dtype, bias), out_global_scale) in one kernel: the
    GEMM epilogue quantizes its tile, the [m, n] tensor never reaches memory.  Returns (uint8 [m, n/2],
    float8_e4m3fn [round_up(m,128), round_up(n/16,4)]), ready to be the `a` operand of the next layer."""
    assert alpha is not None, "alpha must be a CUDA tensor"
    assert value_dtype in (torch.float16, torch.bfloat16), f"value_dtype needs to be fp16 or bf16 but got {value_dtype}"
    _mm_asserts(a, b, block_scale_a, block_scale_b, alpha, value_dtype, torch.float8_e4m3fn)
    assert out_global_scale.is_cuda and out_global_scale.dtype == torch.float, "out_global_scale must be a CUDA fp32 tensor"
    m, n = a.shape[0], b.shape[0]
    assert n % 32 == 0, f"n has to be multiple of 32, but got {n}."
    out = torch.empty((m, n // 2), dtype=torch.uint8, device=a.device)
    out_sf = torch.empty((_round_up(m, 128), _round_up(n // 16, 4) // 4), dtype=torch.int32, device=a.device)
    if bias is not None:
        bias = _check_bias(bias, n, value_dtype)
    ext = _load_scaled_fp4_ops(("scaled_fp4_mm_fp4out",))
    ext.scaled_fp4_mm_fp4out(out, out_sf, a, b, block_scale_a, block_scale_b, alpha, bias, out_global_scale,
                             1 if value_dtype == torch.bfloat16 else 0, False)
    return out, out_sf.view(torch.float8_e4m3fn)


def interleave_gate_up(w_gate: torch.Tensor, w_up: torch.Tensor) -> torch.Tensor:
    """[I, K] gate and up weights -> [2I, K] with rows interleaved in groups of 16 (16 gate rows, their 16 up rows, ...),
    the order scaled_fp4_mm_silu_mul expects.  Quantize the result as one tensor."""
    assert w_gate.shape == w_up.shape and w_gate.ndim == 2 and w_gate.shape[0] % 16 == 0, \
        f"gate and up must be [I, K] with I a multiple of 16, got {tuple(w_gate.shape)} and {tuple(w_up.shape)}"
    i, k = w_gate.shape
    return torch.stack((w_gate.reshape(i // 16, 16, k), w_up.reshape(i // 16, 16, k)), dim=1).reshape(2 * i, k).contiguous()


def scaled_fp4_mm_silu_mul(a, b, block_scale_a, block_scale_b, alpha, value_dtype=torch.bfloat16,
                           out_global_scale=None, bias=None):
    """Gate/up projection of a gated MLP with silu(gate) * up in the GEMM epilogue; `b` is the quantized
    interleave_gate_up(w_gate, w_up).  Returns the [m, n/2] activation in value_dtype, or, with out_global_scale,
    its NVFP4 quantization (uint8 [m, n/4], float8_e4m3fn scales) ready to be the down projection's `a` operand."""
    assert alpha is not None, "alpha must be a CUDA tensor"
    assert value_dtype in (torch.float16, torch.bfloat16), f"value_dtype needs to be fp16 or bf16 but got {value_dtype}"
    _mm_asserts(a, b, block_scale_a, block_scale_b, alpha, value_dtype, torch.float8_e4m3fn)
    m, n = a.shape[0], b.shape[0]
    assert n % 32 == 0, f"n has to be multiple of 32, but got {n}."
    if bias is not None:
        bias = _check_bias(bias, n, value_dtype)
    code = 1 if value_dtype == torch.bfloat16 else 0
    ext = _load_scaled_fp4_ops(("scaled_fp4_mm_silu_mul",))
    if out_global_scale is None:
        out = torch.empty((m, n // 2), dtype=value_dtype, device=a.device)
        ext.scaled_fp4_mm_silu_mul(out, None, a, b, block_scale_a, block_scale_b, alpha, bias, None, code, False)
        return out
    assert out_global_scale.is_cuda and out_global_scale.dtype == torch.float, "out_global_scale must be a CUDA fp32 tensor"
    out = torch.empty((m, n // 4), dtype=torch.uint8, device=a.device)
    out_sf = torch.empty((_round_up(m, 128), _round_up(n // 32, 4) // 4), dtype=torch.int32, device=a.device)
    ext.scaled_fp4_mm_silu_mul(out, out_sf, a, b, block_scale_a, block_scale_b, alpha, bias, out_global_scale, code, False)
    return out, out_sf.view(torch.float8_e4m3fn)


def mxfp4_scaled_mm(a, b, block_scale_a, block_scale_b, out_dtype, alpha=None, bias=None) -> torch.Tensor:
    _mm_asserts(a, b, block_scale_a, block_scale_b, alpha, out_dtype, torch.float8_e8m0fnu)
    m, n = a.shape[0], b.shape[0]
    out = torch.empty((m, n), dtype=out_dtype, device=a.device)
    if bias is not None:
        ext = _load_scaled_fp4_ops(("scaled_fp4_mm_bias",))
        ext.scaled_fp4_mm_bias(out, a, b, block_scale_a, block_scale_b, alpha, _check_bias(bias, n, out_dtype), True)
        return out
    ext = _load_scaled_fp4_ops(("mxfp4_scaled_mm",))
    ext.mxfp4_scaled_mm(out, a, b, block_scale_a, block_scale_b, alpha)
    return out


def global_scale(input: torch.Tensor, scratch: torch.Tensor | None = None) -> torch.Tensor:
    """fp32 [1] on the device: (448*6)/max|input|, without materialising |input|."""
    assert input.is_cuda, "input must be a CUDA tensor"
    assert input.dtype in (torch.float16, torch.bfloat16), f"input.dtype needs to be fp16 or bf16 but got {input.dtype}."
    x = input.reshape(1 if input.ndim == 1 else -1, input.shape[-1])
    assert x.shape[-1] % 8 == 0, f"last dim has to be multiple of 8, but got {x.shape[-1]}."
    if x.stride(-1) != 1 or (x.shape[0] > 1 and x.stride(0) % 8 != 0) or x.data_ptr() % 16 != 0:
        x = x.contiguous()
    out = torch.empty(1, dtype=torch.float32, device=input.device)
    if scratch is None:
        scratch = torch.empty(2, dtype=torch.int32, device=input.device)
    ext = _load_scaled_fp4_ops(("global_scale",))
    ext.global_scale(out, scratch, x)
    return out


def activation_scales(input: torch.Tensor, gs_weight: torch.Tensor, scratch: torch.Tensor):
    """(gs, alpha) = (2688/max|input|, 1/(gs*gs_weight)) in ONE launch.  `scratch`: 8 int32 on the device,
    zeroed once by the caller (torch.zeros) and then reused for every call on the same stream."""
    assert input.is_cuda, "input must be a CUDA tensor"
    assert input.dtype in (torch.float16, torch.bfloat16), f"input.dtype needs to be fp16 or bf16 but got {input.dtype}."
    x = input.reshape(1 if input.ndim == 1 else -1, input.shape[-1])
    assert x.shape[-1] % 8 == 0, f"last dim has to be multiple of 8, but got {x.shape[-1]}."
    if x.stride(-1) != 1 or (x.shape[0] > 1 and x.stride(0) % 8 != 0) or x.data_ptr() % 16 != 0:
        x = x.contiguous()
    out = torch.empty(2, dtype=torch.float32, device=input.device)
    gs, alpha = out[:1], out[1:]
    ext = _load_scaled_fp4_ops(("activation_scales",))
    ext.activation_scales(gs, alpha, scratch, x, gs_weight)
    return gs, alpha


def dynamic_scaled_fp4_quant(input: torch.Tensor, scratch: torch.Tensor, gs_weight: torch.Tensor | None = None):
    """Per-tensor dynamic NVFP4 quantization in one pass over the input:
    (fp4, scales, gs, alpha) with gs = 2688/max|input|, (fp4, scales) = scaled_fp4_quant(input, gs) bit for bit and
    alpha = 1/(gs*gs_weight) (None without gs_weight).  `scratch` as for activation_scales."""
    input, output, output_scale = _quant_common(input, 16)
    out = torch.empty(2, dtype=torch.float32, device=input.device)
    gs, alpha = out[:1], out[1:]
    ext = _load_scaled_fp4_ops(("dynamic_scaled_fp4_quant",))
    ext.dynamic_scaled_fp4_quant(output, output_scale, gs, alpha, scratch, input, gs_weight)
    return output, output_scale.view(torch.float8_e4m3fn), gs, (alpha if gs_weight is not None else None)


def linear_forward(input: torch.Tensor, weight_fp4: torch.Tensor, weight_sf: torch.Tensor,
                   weight_global_scale: torch.Tensor, scratch: torch.Tensor, out_dtype: torch.dtype,
                   bias: torch.Tensor | None = None) -> torch.Tensor:
    """out[m, n] of an NVFP4 layer with online activation quantization (the reference's
    FP4GemmWithOnlineActivation.forward, speed_test.py:43-50) in ONE extension call: global scale, alpha, quantize,
    GEMM (+ bias).  input: [m, k] fp16/bf16; the weight as scaled_fp4_quant produced it."""
    assert input.is_cuda and input.ndim == 2, "input must be a CUDA matrix"
    assert input.dtype in (torch.float16, torch.bfloat16), f"input.dtype needs to be fp16 or bf16 but got {input.dtype}."
    m, k = input.shape
    assert k % 32 == 0, f"last dim has to be multiple of 32, but got {k}."
    if input.stride(-1) != 1 or (m > 1 and input.stride(0) % 8 != 0) or input.data_ptr() % 16 != 0:
        input = input.contiguous()
    n = weight_fp4.shape[0]
    ext = _load_scaled_fp4_ops(("linear_forward", "linear_workspace_bytes"))
    out = torch.empty((m, n), dtype=out_dtype, device=input.device)
    workspace = torch.empty(ext.linear_workspace_bytes(m, k), dtype=torch.uint8, device=input.device)
    if bias is not None:
        bias = _check_bias(bias, n, out_dtype)
    ext.linear_forward(out, input, weight_fp4, weight_sf, weight_global_scale, bias, workspace, scratch)
    return out


def linear_forward_chained(input: torch.Tensor, weight_fp4: torch.Tensor, weight_sf: torch.Tensor,
                           weight_global_scale: torch.Tensor, scratch: torch.Tensor, out_dtype: torch.dtype,
                           bias: torch.Tensor | None = None, input_global_scale: torch.Tensor | None = None,
                           output_scale_scratch: torch.Tensor | None = None,
                           next_weight_global_scale: torch.Tensor | None = None):
    """linear_forward for a layer inside a chain of quantized layers.

    input_global_scale: fp32 [1] on the device, the NVFP4 global scale of `input` when the caller already has it (the
        layer before returned it): the pass over `input` for its maximum is skipped.  None: dynamic, as linear_forward.
    output_scale_scratch: 8 int32 on the device, zeroed once (a buffer of its own, not `scratch`).  Given: the GEMM's
        epilogue also forms the global scale of the OUTPUT, 2688 / max|out|, bit for bit global_scale(out), and, with
        next_weight_global_scale, the next layer's alpha = 1 / (that scale * next_weight_global_scale).
    Returns out, or (out, out_global_scale, next_alpha or None) when output_scale_scratch is given."""
    assert input.is_cuda and input.ndim == 2, "input must be a CUDA matrix"
    assert input.dtype in (torch.float16, torch.bfloat16), f"input.dtype needs to be fp16 or bf16 but got {input.dtype}."
    assert out_dtype in (torch.float16, torch.bfloat16), f"out_dtype needs to be fp16 or bf16 but got {out_dtype}."
    m, k = input.shape
    assert k % 32 == 0, f"last dim has to be multiple of 32, but got {k}."
    if input.stride(-1) != 1 or (m > 1 and input.stride(0) % 8 != 0) or input.data_ptr() % 16 != 0:
        input = input.contiguous()
    n = weight_fp4.shape[0]
    ext = _load_scaled_fp4_ops(("linear_forward_chained", "linear_workspace_bytes"))
    out = torch.empty((m, n), dtype=out_dtype, device=input.device)
    workspace = torch.empty(ext.linear_workspace_bytes(m, k), dtype=torch.uint8, device=input.device)
    if bias is not None:
        bias = _check_bias(bias, n, out_dtype)
    scales = next_alpha = None
    if output_scale_scratch is not None:
        scales = torch.empty(2, dtype=torch.float32, device=input.device)
        next_alpha = scales[1:] if next_weight_global_scale is not None else None
    ext.linear_forward_chained(out, input, input_global_scale, weight_fp4, weight_sf, weight_global_scale, bias, workspace,
                               scratch, scales[:1] if scales is not None else None, output_scale_scratch,
                               next_weight_global_scale, next_alpha)
    if output_scale_scratch is None:
        return out
    return out, scales[:1], next_alpha


def gated_mlp_forward(input: torch.Tensor, gate_up_fp4: torch.Tensor, gate_up_sf: torch.Tensor,
                      gate_up_global_scale: torch.Tensor, down_fp4: torch.Tensor, down_sf: torch.Tensor,
                      act_global_scale: torch.Tensor, down_alpha: torch.Tensor, scratch: torch.Tensor,
                      out_dtype: torch.dtype) -> torch.Tensor:
    """down(silu(gate(x)) * up(x)) with NVFP4 weights in ONE extension call (three chained launches: quantizer,
    gate/up GEMM with activation and quantizer in its epilogue, down GEMM).  gate_up: rows interleaved with
    interleave_gate_up and quantized as one tensor; act_global_scale: calibrated scale of the hidden activation;
    down_alpha = alpha_from_scales(act_global_scale, down weight's global scale).  Same bytes as
    dynamic_scaled_fp4_quant -> scaled_fp4_mm_silu_mul(out_global_scale=...) -> cutlass_scaled_fp4_mm."""
    assert input.is_cuda and input.ndim == 2, "input must be a CUDA matrix"
    assert input.dtype in (torch.float16, torch.bfloat16), f"input.dtype needs to be fp16 or bf16 but got {input.dtype}."
    assert out_dtype in (torch.float16, torch.bfloat16), f"out_dtype needs to be fp16 or bf16 but got {out_dtype}."
    m, hidden = input.shape
    if input.stride(-1) != 1 or (m > 1 and input.stride(0) % 8 != 0) or input.data_ptr() % 16 != 0:
        input = input.contiguous()
    inter = gate_up_fp4.shape[0] // 2
    ext = _load_scaled_fp4_ops(("gated_mlp_forward", "gated_mlp_workspace_bytes"))
    out = torch.empty((m, down_fp4.shape[0]), dtype=out_dtype, device=input.device)
    workspace = torch.empty(ext.gated_mlp_workspace_bytes(m, hidden, inter), dtype=torch.uint8, device=input.device)
    ext.gated_mlp_forward(out, input, gate_up_fp4, gate_up_sf, gate_up_global_scale, down_fp4, down_sf,
                          act_global_scale, down_alpha, workspace, scratch)
    return out


def alpha_from_scales(gs_a: torch.Tensor, gs_b: torch.Tensor) -> torch.Tensor:
    out = torch.empty(1, dtype=torch.float32, device=gs_a.device)
    ext = _load_scaled_fp4_ops(("alpha_from_scales",))
    ext.alpha_from_scales(out, gs_a, gs_b)
    return out
