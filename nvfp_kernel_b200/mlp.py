"""QuantGatedMLP: down(silu(gate(x)) * up(x)) with NVFP4 weights in three launches (one extension call).

    quantize x (global scale of x, alpha, NVFP4 bytes: one pass)
    gate/up GEMM whose epilogue applies silu(gate) * up and quantizes the result for the down projection
    down GEMM

The gate and up weights are kept as one tensor with rows interleaved in groups of 16 (ops.interleave_gate_up), so the
GEMM epilogue finds each gate value next to its up value; the hidden activation never exists as a 16-bit tensor.  Its
global scale cannot be computed on the fly (it would need the maximum of a tensor that is never materialised), so it
is a calibrated constant: `calibrate(x)` measures it on sample inputs, as deployment recipes for NVFP4 do.

Tensor parallel (`parallel="tensor"`): the intermediate dimension is split over the ranks, gate/up column-parallel and
down row-parallel on the same shard, so nothing is exchanged between the two GEMMs; the down projection's partial
sums are reduce-scattered over the rows, by NCCL or (`fused_reduce_scatter=True`) by the GEMM epilogue adding its
tiles into the owning rank's buffer over NVLink.  The reference has no such module; its pieces are
FP4GemmWithOnlineActivation (speed_test.py:36-50 there).
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import ops
from .sharding import shard_columns, shard_range, shard_rows


class QuantGatedMLP(nn.Module):
    def __init__(self, hidden_size: int, intermediate_size: int, parallel: str | None = None, process_group=None,
                 out_dtype: torch.dtype = torch.bfloat16, fused_reduce_scatter: bool = False, device=None):
        super().__init__()
        if parallel not in (None, "tensor"):
            raise ValueError(f"parallel={parallel!r}; expected None or 'tensor'")
        if out_dtype not in (torch.float16, torch.bfloat16):
            raise ValueError(f"out_dtype={out_dtype}; expected torch.float16 or torch.bfloat16")
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.parallel, self.process_group, self.out_dtype = parallel, process_group, out_dtype
        self.fused_reduce_scatter = fused_reduce_scatter and parallel is not None
        self._reduce_buffers = {}
        self.world, self.rank = 1, 0
        if parallel is not None:
            import torch.distributed as dist
            self.world, self.rank = dist.get_world_size(process_group), dist.get_rank(process_group)
        # 64: the K granule of the down projection's shard (whole scale tiles) and half the row granule of the
        # interleaved gate/up shard (128 rows)
        lo, hi = shard_range(intermediate_size, self.rank, self.world, 64, "intermediate_size")
        self.inter_local = il = hi - lo
        rows = lambda n: (n + 127) // 128 * 128
        cols = lambda k: (k // 16 + 3) // 4 * 4
        self.register_buffer("gate_up_fp4", torch.zeros((2 * il, hidden_size // 2), dtype=torch.uint8, device=device))
        self.register_buffer("gate_up_sf", torch.zeros((rows(2 * il), cols(hidden_size)), dtype=torch.uint8, device=device))
        self.register_buffer("gate_up_global_scale", torch.ones(1, dtype=torch.float32, device=device))
        self.register_buffer("down_fp4", torch.zeros((hidden_size, il // 2), dtype=torch.uint8, device=device))
        self.register_buffer("down_sf", torch.zeros((rows(hidden_size), cols(il)), dtype=torch.uint8, device=device))
        self.register_buffer("down_global_scale", torch.ones(1, dtype=torch.float32, device=device))
        # global scale of silu(gate) * up and the down GEMM's alpha = 1 / (act_global_scale * down_global_scale)
        self.register_buffer("act_global_scale", torch.ones(1, dtype=torch.float32, device=device))
        self.register_buffer("down_alpha", torch.ones(1, dtype=torch.float32, device=device))
        self.register_buffer("_scale_scratch", torch.zeros(8, dtype=torch.int32, device=device), persistent=False)

    # ------------------------------------------------------------------ weights ---
    @torch.no_grad()
    def load_weights(self, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor) -> "QuantGatedMLP":
        """Quantizes the FULL fp16/bf16 weights (gate, up: [intermediate, hidden]; down: [hidden, intermediate]) on
        their device with full-tensor global scales and keeps this rank's shard."""
        inter, hidden = self.intermediate_size, self.hidden_size
        assert w_gate.shape == (inter, hidden) and w_up.shape == (inter, hidden) and w_down.shape == (hidden, inter), \
            "weight shape mismatch"
        w_gu = ops.interleave_gate_up(w_gate, w_up)
        gs = ops.global_scale(w_gu)
        gu_fp4, gu_sf = ops.scaled_fp4_quant(w_gu, gs)
        self.gate_up_global_scale.copy_(gs)
        gs = ops.global_scale(w_down)
        d_fp4, d_sf = ops.scaled_fp4_quant(w_down, gs)
        self.down_global_scale.copy_(gs)
        gu_sf, d_sf = gu_sf.view(torch.uint8), d_sf.view(torch.uint8)
        if self.world > 1:
            gu_fp4, gu_sf = shard_columns(gu_fp4, gu_sf, self.rank, self.world)
            d_fp4, d_sf = shard_rows(d_fp4, d_sf, self.rank, self.world, 16)
        dev = self.gate_up_fp4.device
        self.gate_up_fp4, self.gate_up_sf = gu_fp4.to(dev), gu_sf.to(dev)
        self.down_fp4, self.down_sf = d_fp4.to(dev), d_sf.to(dev)
        self.set_activation_scale(self.act_global_scale)
        return self

    @torch.no_grad()
    def set_activation_scale(self, act_global_scale: torch.Tensor) -> "QuantGatedMLP":
        """Global scale (2688 / expected max) of the hidden activation silu(gate) * up."""
        self.act_global_scale.copy_(act_global_scale.reshape(1).to(torch.float32))
        self.down_alpha.copy_(ops.alpha_from_scales(self.act_global_scale, self.down_global_scale))
        return self

    @torch.no_grad()
    def calibrate(self, x: torch.Tensor, margin: float = 1.0) -> "QuantGatedMLP":
        """Sets the hidden activation's scale from sample inputs: 2688 / (margin * max|silu(gate) * up|), the maximum
        taken over all ranks' shards."""
        h = self._hidden_16bit(x.reshape(-1, x.shape[-1]))
        amax = h.float().abs().max().reshape(1)
        if self.world > 1:
            import torch.distributed as dist
            dist.all_reduce(amax, op=dist.ReduceOp.MAX, group=self.process_group)
        amax = torch.where(amax == 0, torch.ones_like(amax), amax) * margin
        return self.set_activation_scale((448.0 * 6.0) / amax)

    def _sf(self, t: torch.Tensor) -> torch.Tensor:
        return t.view(torch.float8_e4m3fn)

    def _hidden_16bit(self, x2: torch.Tensor) -> torch.Tensor:
        x_fp4, x_sf, _, alpha = ops.dynamic_scaled_fp4_quant(x2, self._scale_scratch, self.gate_up_global_scale)
        return ops.scaled_fp4_mm_silu_mul(x_fp4, self.gate_up_fp4, x_sf, self._sf(self.gate_up_sf), alpha, self.out_dtype)

    # ------------------------------------------------------------------ forward ---
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """[..., hidden] -> [..., hidden]; tensor parallel: [M / world, hidden], this rank's rows of the result (the
        whole [M, hidden] when M is not a multiple of the world size)."""
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1])
        if self.world == 1:
            # one extension call; the three launches are chained so that each GEMM streams its weights under the
            # kernel before it
            y = ops.gated_mlp_forward(x2, self.gate_up_fp4, self.gate_up_sf, self.gate_up_global_scale, self.down_fp4,
                                      self.down_sf, self.act_global_scale, self.down_alpha, self._scale_scratch,
                                      self.out_dtype)
            return y.reshape(*lead, self.hidden_size)
        x_fp4, x_sf, _, alpha = ops.dynamic_scaled_fp4_quant(x2, self._scale_scratch, self.gate_up_global_scale)
        h_fp4, h_sf = ops.scaled_fp4_mm_silu_mul(x_fp4, self.gate_up_fp4, x_sf, self._sf(self.gate_up_sf), alpha,
                                                 self.out_dtype, out_global_scale=self.act_global_scale)
        return self._down_reduce(h_fp4, h_sf)

    def _down_reduce(self, h_fp4: torch.Tensor, h_sf: torch.Tensor) -> torch.Tensor:
        import torch.distributed as dist
        from ._ops_real import _load_scaled_fp4_ops
        m = h_fp4.shape[0]
        if self.fused_reduce_scatter and m % (32 * self.world) == 0:
            from .peer import ReduceBuffer
            rb = self._reduce_buffers.get(m)
            if rb is None:
                rb = self._reduce_buffers[m] = ReduceBuffer(m, self.hidden_size, h_fp4.device, self.process_group)
            # the kernel synchronises the ranks itself: it announces "ready" when it starts (after this zeroing, in
            # stream order) and ends when every rank's contributions have arrived
            rb.buf.zero_()
            _load_scaled_fp4_ops(("scaled_fp4_mm_reduce_scatter",)).scaled_fp4_mm_reduce_scatter(
                rb.dst_ptrs, rb.flag_ptrs, rb.rank, rb.wait_limit_ns, h_fp4, self.down_fp4, h_sf.view(torch.uint8),
                self.down_sf, self.down_alpha, False)
            return rb.buf.to(self.out_dtype)
        part = torch.empty((m, self.hidden_size), dtype=torch.float32, device=h_fp4.device)
        _load_scaled_fp4_ops(("cutlass_scaled_fp4_mm",)).cutlass_scaled_fp4_mm(
            part, h_fp4, self.down_fp4, h_sf, self._sf(self.down_sf), self.down_alpha)
        if m % self.world != 0:
            dist.all_reduce(part, group=self.process_group)
            return part.to(self.out_dtype)
        out = torch.empty((m // self.world, self.hidden_size), dtype=torch.float32, device=part.device)
        dist.reduce_scatter_tensor(out, part, group=self.process_group)
        return out.to(self.out_dtype)

    def reference_forward(self, x: torch.Tensor) -> torch.Tensor:
        """The same layer with separate kernels (16-bit hidden activation, dynamic scale): for comparisons."""
        assert self.world == 1, "single-GPU helper"
        x2 = x.reshape(-1, x.shape[-1])
        h = self._hidden_16bit(x2)
        h_fp4, h_sf, _, alpha = ops.dynamic_scaled_fp4_quant(h, self._scale_scratch, self.down_global_scale)
        return ops.cutlass_scaled_fp4_mm(h_fp4, self.down_fp4, h_sf, self._sf(self.down_sf), alpha, self.out_dtype)

    def extra_repr(self) -> str:
        return (f"hidden_size={self.hidden_size}, intermediate_size={self.intermediate_size}, parallel={self.parallel}, "
                f"world={self.world}")


def dense_gated_mlp(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor) -> torch.Tensor:
    """Unquantized reference: down(silu(gate(x)) * up(x)) in the tensors' own dtype."""
    return F.linear(F.silu(F.linear(x, w_gate)) * F.linear(x, w_up), w_down)
