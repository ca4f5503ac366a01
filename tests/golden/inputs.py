"""Seeded synthetic inputs shared by the fixture generators and the tests.

All tensors are drawn from a CPU ``torch.Generator`` so that the CPU oracle and the
GPU kernels see identical bits.  The seven distributions restate the reference's
``DataGenerator.get_random_tensor`` (emulation/utils.py:38-59).
"""
import math

import torch

DISTRIBUTIONS = ("normal", "uniform", "large", "small", "outliers", "mixed_rows", "abs_large")


def make_input(dist: str, shape, dtype=torch.bfloat16, seed: int = 0) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    randn = lambda s: torch.randn(s, generator=g, dtype=torch.float32)
    if dist == "normal":
        t = randn(shape)
    elif dist == "uniform":
        t = torch.rand(shape, generator=g) * 2 - 1
    elif dist == "large":
        t = randn(shape) * 100.0
    elif dist == "small":
        t = randn(shape) * 0.001
    elif dist == "outliers":
        t = randn(shape)
        mask = torch.rand(shape, generator=g) < 0.01
        t[mask] *= 50.0
    elif dist == "mixed_rows":
        t = randn(shape) * torch.exp(randn((shape[0], 1)) * 2)
    elif dist == "abs_large":
        t = randn(shape).abs() * 100.0
    elif dist == "zeros_mixed":          # not in the reference: all-zero and denormal blocks
        t = randn(shape)
        t[:, : shape[1] // 4] = 0.0
        t[:, shape[1] // 4: shape[1] // 2] *= 1e-38
    elif dist == "specials":             # not in the reference: infinities, NaNs, -0, denormals, the largest finite value
        t = randn(shape).to(dtype)
        fi = torch.finfo(dtype)
        values = [float("inf"), -float("inf"), float("nan"), -0.0, fi.smallest_normal / 4, -fi.smallest_normal / 8,
                  fi.max, -fi.max, 0.0]
        rows, cols = shape
        for i, v in enumerate(values):
            t[(3 + 7 * i) % rows, (5 + 16 * i) % cols] = v                       # one special value in an ordinary block
            c0 = (16 * (i % max(1, cols // 16))) % cols
            t[(40 + i) % rows, c0: c0 + 16] = v                                  # a block of nothing else
            t[(60 + i) % rows, c0: c0 + 16: 2] = v                               # every other element of a block
        return t
    elif dist == "student_t3":           # BASELINE config 5 activations
        z = randn(shape)
        chi2 = (randn(shape) ** 2 + randn(shape) ** 2 + randn(shape) ** 2) / 3.0
        t = z / chi2.sqrt()
    else:
        raise ValueError(dist)
    return t.to(dtype)


def c1_inputs():
    """BASELINE config 1: A [1024,1024] ~N(0,1), W [1024,1024] ~N(0,1/sqrt(K)), bf16,
    seed 0, A then W from the same generator."""
    g = torch.Generator().manual_seed(0)
    a = torch.randn((1024, 1024), generator=g, dtype=torch.float32).to(torch.bfloat16)
    w = (torch.randn((1024, 1024), generator=g, dtype=torch.float32) / math.sqrt(1024)).to(torch.bfloat16)
    return a, w


def gemm_inputs(m: int, n: int, k: int, seed: int = 0, w_std: float = 1.0, dtype=torch.bfloat16,
                outlier_cols: bool = False):
    """Activations ~N(0,1) [m,k] (optionally 1% of K-channels x50) and weights
    ~N(0,w_std) [n,k]."""
    g = torch.Generator().manual_seed(seed)
    a = torch.randn((m, k), generator=g, dtype=torch.float32)
    if outlier_cols:
        g2 = torch.Generator().manual_seed(2)
        mask = torch.rand((k,), generator=g2) < 0.01
        a[:, mask] *= 50.0
    g1 = torch.Generator().manual_seed(seed + 1)
    w = torch.randn((n, k), generator=g1, dtype=torch.float32) * w_std
    return a.to(dtype), w.to(dtype)


def mx_duplicated_halves(dist: str, shape, dtype=torch.bfloat16, seed: int = 17) -> torch.Tensor:
    """[m, n] input whose every 32-element block is two copies of one 16-element half: a 16-block quantizer (the
    reference's e8m0 branch) and a 32-block quantizer (MXFP4 here) must then choose the same scale for it."""
    m, n = shape
    half = make_input(dist, (m, n // 2), dtype, seed).reshape(m, n // 32, 1, 16)
    return half.expand(m, n // 32, 2, 16).reshape(m, n).contiguous()
