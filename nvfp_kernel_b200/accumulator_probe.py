"""How wide is the accumulator of the block-scaled FP4 MMA?  A probe with exact inputs.

    python -m nvfp_kernel_b200.accumulator_probe

The reference spends a whole sub-project (its emulation/ directory, AGENTS.md:27-58 there) on finding the alignment
width and rounding of the sm_120 tensor core by search.  With exact inputs the question can be put to the hardware
directly: one output element is the sum of a BIG product 2^e and one or more SMALL products 2^(e-s); every term is a
power of two (e2m1 value 1.0 times power-of-two block scales), so the exact sum is known, and what the GEMM returns
shows how many bits below the largest term survive, and whether what does not survive is rounded or dropped.

Placements of the small term(s) relative to the big one:
    block      another 16-element block of the same 64-element MMA (K offset 16)
    mma        the next MMA instruction (K offset 64), accumulated into the same tensor-memory word
    15 block   15 small terms 2^(e-s) in one other block of the same MMA (their exact sum is 15 * 2^(e-s))
    15 mma     the same 15 terms in the next MMA instruction
    15 neg     as "15 block" with every term negative: tells truncation (toward zero) from rounding down

Result on B200 (tcgen05.mma kind::mxf4nvf4, fp32 accumulator in tensor memory): a single term survives down to
s = 23 and not at 24; fifteen terms give 15, 15, ..., 15 (s <= 23), 14 (s = 24), 12, 8, 0 -- the exact sum
big + 15 * small CHOPPED to the 24 bits below the big term's leading bit (round to nearest would give 16, 16, 8).  The
terms of one instruction are therefore added exactly (at least 4 bits below the fp32 ulp are carried) and the sum is
truncated toward zero once; the same holds when the small terms arrive with the next instruction, and for negative
sums.  The CPU oracle's fp64 dot product differs from this by at most one fp32 ulp per accumulation step, far inside the
1e-2 tolerance of the GEMM tests.
"""
from __future__ import annotations

import torch

from . import ops

_E2M1_ONE = 0x2                     # e2m1 code of 1.0


def _e4m3_pow2(p: int) -> int:
    """ue4m3 byte of 2^p, p in [-9, 8] (denormals below 2^-6)."""
    if p >= -6:
        return (p + 7) << 3
    return 1 << (p + 9)


def _swizzled_scales(rows: int, k: int, values: dict) -> torch.Tensor:
    """Scale tensor [round_up(rows,128), round_up(k/16,4)] in the [rowTile][kTile][32][4][4] byte order, all 2^0
    except `values[(row, block)] = byte`."""
    rp, cp = (rows + 127) // 128 * 128, (k // 16 + 3) // 4 * 4
    flat = torch.full((rp * cp,), _e4m3_pow2(0), dtype=torch.uint8)
    k_tiles = cp // 4
    for (row, blk), byte in values.items():
        off = ((row // 128) * k_tiles + blk // 4) * 512 + (row % 32) * 16 + ((row % 128) // 32) * 4 + blk % 4
        flat[off] = byte
    return flat.view(rp, cp)


def _run(terms, m: int = 128, n: int = 128, k: int = 128, negative: bool = False) -> float:
    """terms: list of (k_index, pa, pb): a[0, k_index] = b[0, k_index] = 1.0 (a = -1.0 if negative) with block
    scales 2^pa and 2^pb.  Returns out[0, 0] in fp32."""
    a = torch.zeros((m, k // 2), dtype=torch.uint8)
    b = torch.zeros((n, k // 2), dtype=torch.uint8)
    sa, sb = {}, {}
    for kk, pa, pb in terms:
        shift = 4 * (kk % 2)
        a[0, kk // 2] |= (_E2M1_ONE | (0x8 if negative else 0)) << shift
        b[0, kk // 2] |= _E2M1_ONE << shift
        sa[(0, kk // 16)] = _e4m3_pow2(pa)
        sb[(0, kk // 16)] = _e4m3_pow2(pb)
    sfa = _swizzled_scales(m, k, sa).cuda().view(torch.float8_e4m3fn)
    sfb = _swizzled_scales(n, k, sb).cuda().view(torch.float8_e4m3fn)
    alpha = torch.ones(1, device="cuda")
    from ._ops_real import _load_scaled_fp4_ops
    out = torch.empty((m, n), dtype=torch.float32, device="cuda")
    _load_scaled_fp4_ops(("cutlass_scaled_fp4_mm",)).cutlass_scaled_fp4_mm(out, a.cuda(), b.cuda(), sfa, sfb, alpha)
    return float(out[0, 0].item())


def _split(e: int):
    """2^e as a product of two representable block scales 2^pa * 2^pb."""
    pa = max(-9, min(8, e // 2))
    return pa, e - pa


BIG_E = 16                                                  # big term 2^16 = (2^8 scale) * (2^8 scale)
PLACEMENTS = ("block", "mma", "15 block", "15 mma", "15 neg")


def measure(s: int) -> dict:
    """(result - big) in units of the small term 2^(BIG_E - s), for every placement."""
    e = BIG_E - s
    pa, pb = _split(e)
    big, unit = float(2 ** BIG_E), float(2.0 ** e)
    return {
        "block": (_run([(0, 8, 8), (16, pa, pb)]) - big) / unit,
        "mma": (_run([(0, 8, 8), (64, pa, pb)]) - big) / unit,
        "15 block": (_run([(0, 8, 8)] + [(16 + i, pa, pb) for i in range(15)]) - big) / unit,
        "15 mma": (_run([(0, 8, 8)] + [(64 + i, pa, pb) for i in range(15)]) - big) / unit,
        "15 neg": (-_run([(0, 8, 8)] + [(16 + i, pa, pb) for i in range(15)], negative=True) - big) / unit,
    }


def truncation_model(count: int, s: int) -> int:
    """What `measure` returns if the `count` small terms are added to the big one EXACTLY and the sum is then
    truncated toward zero to fp32's 24 significant bits: one fp32 ulp of the big term is 2^(s-23) small units."""
    if s <= 23:
        return count
    step = 1 << (s - 23)
    return count // step * step


def main():
    assert ops.get_active_backend() == "real"
    print(f"big term 2^{BIG_E}; small term(s) 2^({BIG_E}-s); entries = (result - big) in units of the small term")
    print(f"{'s':>3} {'block':>8} {'mma':>8} {'15 block':>9} {'15 mma':>8} {'15 neg':>8}")
    for s in range(20, 30):
        r = measure(s)
        print(f"{s:>3} {r['block']:>8.0f} {r['mma']:>8.0f} {r['15 block']:>9.0f} {r['15 mma']:>8.0f} {r['15 neg']:>8.0f}")
    print("fp32 itself keeps s <= 23 exactly (24-bit significand); s = 24 is the round-to-nearest-even tie.")


if __name__ == "__main__":
    main()
