"""Swap the nn.Linear layers of a model for QuantLinear(mode="real").

The reference's log of a llama-2-7b run (tmp.log:1-7 there) shows a driver script, absent from its
tree, doing exactly this before generation; this is that helper for the B200 path.
"""
from __future__ import annotations

from typing import Callable, Iterable

import torch.nn as nn

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
            q = QuantLinear.from_linear(child, format=format)
            if cuda_graph:
                q.enable_cuda_graph()
            setattr(module, child_name, q)
            replaced.append(full)
    return replaced
