"""Swap the nn.Linear layers of a model for QuantLinear(mode="real"), and its gated MLP blocks for QuantGatedMLP.

The reference's log of a llama-2-7b run (tmp.log:1-7 there) shows a driver script, absent from its
tree, doing exactly this before generation; this is that helper for the B200 path.
"""
from __future__ import annotations

from typing import Callable, Iterable

import torch.nn as nn

import torch

from .linear import QuantLinear


def quantize_linear_layers(model: nn.Module, format: str = "nvfp4", skip: Iterable[str] = ("lm_head",),
                           predicate: Callable[[str, nn.Linear], bool] | None = None,
                           cuda_graph: bool = False) -> list[str]:
    """Replaces, in place, every nn.Linear on a CUDA device whose in_features is a multiple of the
    format's alignment (32 for nvfp4, 64 for mxfp4) and whose out_features is a multiple of 32.
    `skip`: substrings of module names to leave alone.  Returns the names that were replaced."""
    align = 32 if format == "nvfp4" else 64
    replaced = []
    for name, module in list(model.named_modules()):
        for child_name, child in list(module.named_children()):
            full = f"{name}.{child_name}" if name else child_name
            if not isinstance(child, nn.Linear) or any(s in full for s in skip):
                continue
            if child.in_features % align or child.out_features % 32 or not child.weight.is_cuda:
                continue
            if predicate is not None and not predicate(full, child):
                continue
            # the replacement computes in the model's own 16-bit dtype (an fp16 model keeps fp16 activations; the
            # reference's logged run is fp16, tmp.log:1-7 there); other dtypes get bf16
            out_dtype = child.weight.dtype if child.weight.dtype in (torch.float16, torch.bfloat16) else torch.bfloat16
            q = QuantLinear.from_linear(child, format=format, out_dtype=out_dtype)
            if cuda_graph:
                q.enable_cuda_graph()
            setattr(module, child_name, q)
            replaced.append(full)
    return replaced


def _is_silu(mlp: nn.Module) -> bool:
    act = getattr(mlp, "act_fn", None)
    if act is None:
        return False
    name = (getattr(act, "__name__", "") or type(act).__name__).lower()
    return isinstance(act, nn.SiLU) or "silu" in name or "swish" in name


def quantize_gated_mlps(model: nn.Module, run_calibration: Callable[[], None], margin: float = 1.0,
                        skip: Iterable[str] = (), proj_names=("gate_proj", "up_proj", "down_proj")) -> list[str]:
    """Replaces, in place, every block of the form down_proj(silu(gate_proj(x)) * up_proj(x)) (three bias-free
    nn.Linear children with those names and an `act_fn` that is SiLU, as in Llama-style models) with a QuantGatedMLP:
    three launches per block, the hidden activation never materialised.

    The hidden activation's NVFP4 global scale has to be known before the block runs, so it is calibrated:
    `run_calibration()` must run the (still unquantized) model on representative inputs; the largest |input| that each
    block's down projection sees becomes that block's scale (2688 / (margin * max)).  Returns the replaced names."""
    from .mlp import QuantGatedMLP
    gate_n, up_n, down_n = proj_names
    targets = []
    for name, module in list(model.named_modules()):
        for child_name, child in list(module.named_children()):
            full = f"{name}.{child_name}" if name else child_name
            projs = [getattr(child, n, None) for n in proj_names]
            if not all(isinstance(p, nn.Linear) and p.bias is None and p.weight.is_cuda for p in projs):
                continue
            if any(s in full for s in skip) or not _is_silu(child):
                continue
            gate, up, down = projs
            hidden, inter = gate.in_features, gate.out_features
            if (up.in_features, up.out_features) != (hidden, inter) or (down.in_features, down.out_features) != (inter, hidden):
                continue
            if hidden % 32 or inter % 64 or gate.weight.dtype not in (torch.float16, torch.bfloat16):
                continue
            targets.append((module, child_name, child, full))
    seen, hooks = [], []
    for _, _, mlp, _ in targets:
        amax = torch.zeros(1, dtype=torch.float32, device=getattr(mlp, down_n).weight.device)
        seen.append(amax)

        def record(mod, args, amax=amax):
            amax.copy_(torch.maximum(amax, args[0].detach().abs().max().float().reshape(1)))

        hooks.append(getattr(mlp, down_n).register_forward_pre_hook(record))
    try:
        if targets:
            with torch.no_grad():
                run_calibration()
    finally:
        for h in hooks:
            h.remove()
    replaced = []
    for (parent, child_name, mlp, full), amax in zip(targets, seen):
        if float(amax) == 0.0:
            continue                       # the calibration run never reached this block
        gate, up, down = (getattr(mlp, n) for n in proj_names)
        q = QuantGatedMLP(gate.in_features, gate.out_features, out_dtype=gate.weight.dtype, device=gate.weight.device)
        q.load_weights(gate.weight.data, up.weight.data, down.weight.data)
        q.set_activation_scale((448.0 * 6.0) / (amax * margin))
        setattr(parent, child_name, q)
        replaced.append(full)
    return replaced
