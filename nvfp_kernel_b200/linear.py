"""QuantLinear(mode="real"): a linear layer whose forward runs activation quantize ->
block-scaled FP4 GEMM on the sm_100a kernels.

The reference names this class only in prose (README.md:18 there); the behaviour it
exercises is FP4GemmWithOnlineActivation (speed_test.py:36-50): the weight is quantized
once with gs_w = 2688/max|W|; each call computes gs_a = 2688/max|x|, quantizes x,
forms alpha = 1/(gs_a*gs_w) on the device and calls the GEMM.  This class keeps those
numerics and adds MXFP4 and the two tensor-parallel shardings (see sharding.py).
"""
from __future__ import annotations

import torch
import torch.nn as nn

from . import ops
from .sharding import gather_columns_layout, shard_columns, shard_range, shard_rows

_FORMATS = {"nvfp4": 16, "mxfp4": 32}


class QuantLinear(nn.Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = False, mode: str = "real",
                 format: str = "nvfp4", parallel: str | None = None, process_group=None,
                 out_dtype: torch.dtype = torch.bfloat16, mx_rounding: str = "rceil",
                 gather_output: bool = True, input_is_parallel: bool = False, fused_gather: bool = False,
                 fused_reduce_scatter: bool = False, device=None):
        super().__init__()
        if mode != "real":
            raise ValueError(f"mode={mode!r}: only the real-kernel path exists (no emulation, no pseudo-quant fallback)")
        if format not in _FORMATS:
            raise ValueError(f"format={format!r}; expected one of {sorted(_FORMATS)}")
        if parallel not in (None, "column", "row"):
            raise ValueError(f"parallel={parallel!r}; expected None, 'column' or 'row'")
        self.in_features, self.out_features = in_features, out_features
        self.format, self.block = format, _FORMATS[format]
        self.parallel, self.process_group = parallel, process_group
        self.out_dtype, self.mx_rounding = out_dtype, mx_rounding
        self.gather_output, self.input_is_parallel = gather_output, input_is_parallel
        # column-parallel only: the GEMM epilogue writes this rank's slab into every rank's gathered
        # buffer over NVLink instead of running an all-gather afterwards (see peer.py)
        self.fused_gather = fused_gather and parallel == "column"
        self._gather_buffers = {}
        self._use_graph, self._graphs = False, {}
        # row-parallel only: partial products are added straight into the owning rank's fp32 buffer by the
        # GEMM epilogue (TMA reduce over NVLink) instead of an NCCL reduce-scatter afterwards
        self.fused_reduce_scatter = fused_reduce_scatter and parallel == "row"
        self._reduce_buffers = {}
        # bound (ns) of each in-kernel wait on a peer rank in the fused collectives; 0 = the library's two seconds
        self.peer_wait_limit_ns = 0
        self.world, self.rank = 1, 0
        if parallel is not None:
            import torch.distributed as dist
            self.world = dist.get_world_size(process_group)
            self.rank = dist.get_rank(process_group)
        n_local, k_local = out_features, in_features
        if parallel == "column":
            lo, hi = shard_range(out_features, self.rank, self.world, 128, "out_features")
            n_local = hi - lo
        elif parallel == "row":
            lo, hi = shard_range(in_features, self.rank, self.world, 4 * self.block, "in_features")
            k_local = hi - lo
        self.n_local, self.k_local = n_local, k_local
        rn = (n_local + 127) // 128 * 128
        rk = (k_local // self.block + 3) // 4 * 4
        self.register_buffer("weight_fp4", torch.zeros((n_local, k_local // 2), dtype=torch.uint8, device=device))
        self.register_buffer("weight_sf", torch.zeros((rn, rk), dtype=torch.uint8, device=device))
        self.register_buffer("weight_global_scale", torch.ones(1, dtype=torch.float32, device=device))
        # scratch of the fused amax -> (global scale, alpha) kernel: zeroed once, self-cleaning afterwards
        self.register_buffer("_scale_scratch", torch.zeros(8, dtype=torch.int32, device=device), persistent=False)
        self.bias = nn.Parameter(torch.zeros(out_features, dtype=out_dtype, device=device)) if bias else None

    # ------------------------------------------------------------------ weights ---
    @torch.no_grad()
    def load_weight(self, weight: torch.Tensor) -> "QuantLinear":
        """Quantizes the FULL [out_features, in_features] fp16/bf16 weight on its device
        and keeps this rank's shard."""
        assert weight.shape == (self.out_features, self.in_features), "weight shape mismatch"
        if self.format == "nvfp4":
            gs = ops.global_scale(weight)
            w_fp4, w_sf = ops.scaled_fp4_quant(weight, gs)
            self.weight_global_scale.copy_(gs)
        else:
            w_fp4, w_sf = ops.scaled_mxfp4_quant(weight, self.mx_rounding)
        w_sf = w_sf.view(torch.uint8)
        if self.parallel == "column":
            w_fp4, w_sf = shard_columns(w_fp4, w_sf, self.rank, self.world)
        elif self.parallel == "row":
            w_fp4, w_sf = shard_rows(w_fp4, w_sf, self.rank, self.world, self.block)
        self.weight_fp4 = w_fp4.to(self.weight_fp4.device)
        self.weight_sf = w_sf.to(self.weight_sf.device)
        return self

    @classmethod
    def from_linear(cls, linear: nn.Linear, **kw) -> "QuantLinear":
        w = linear.weight.detach()
        if w.dtype not in (torch.float16, torch.bfloat16):
            w = w.to(torch.bfloat16)
        layer = cls(linear.in_features, linear.out_features, bias=linear.bias is not None,
                    device=w.device, **kw)
        layer.load_weight(w)
        if linear.bias is not None:
            layer.bias.data.copy_(linear.bias.detach().to(layer.bias.dtype))
        return layer

    def _sf_view(self, t: torch.Tensor) -> torch.Tensor:
        return t.view(torch.float8_e4m3fn if self.format == "nvfp4" else torch.float8_e8m0fnu)

    # -------------------------------------------------------------- CUDA graphs ---
    def enable_cuda_graph(self, enabled: bool = True) -> "QuantLinear":
        """Replay one captured CUDA graph per input shape instead of launching the forward's kernels
        one by one (small, launch-bound shapes: the reference's forward has a 40 us floor from 8 launches,
        README.md:34-37 there).  The result aliases a buffer owned by the layer and is overwritten by the
        next call with the same shape.  Not available for tensor-parallel layers."""
        if enabled and self.parallel is not None:
            raise ValueError("CUDA-graph replay is only offered for single-GPU layers")
        self._use_graph = enabled
        if not enabled:
            self._graphs = {}
        return self

    def graph_input(self, shape, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
        """The buffer the graph for this input shape reads.  A caller that writes its activation there and passes
        this very tensor to forward() saves the copy forward() would otherwise make."""
        return self._graph_entry(tuple(shape), dtype, None)[1]

    def _graph_entry(self, shape, dtype, x):
        key = (shape, dtype)
        entry = self._graphs.get(key)
        if entry is None:
            device = self.weight_fp4.device
            static_in = torch.zeros(shape, dtype=dtype, device=device)
            if x is not None:
                static_in.copy_(x)
            stream = torch.cuda.Stream(device=device)
            stream.wait_stream(torch.cuda.current_stream(device))
            with torch.cuda.stream(stream):
                for _ in range(2):                     # warm-up outside capture (lazy initialisation, allocator)
                    self._forward_impl(static_in)
            torch.cuda.current_stream(device).wait_stream(stream)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                static_out = self._forward_impl(static_in)
            entry = self._graphs[key] = (graph, static_in, static_out)
        return entry

    def _graphed_forward(self, x: torch.Tensor) -> torch.Tensor:
        graph, static_in, static_out = self._graph_entry(tuple(x.shape), x.dtype, x)
        if x.data_ptr() != static_in.data_ptr():
            static_in.copy_(x)
        graph.replay()
        return static_out

    # ------------------------------------------------------------------ forward ---
    def forward(self, x: torch.Tensor, x_global_scale: torch.Tensor | None = None, return_output_scale: bool = False,
                next_layer: "QuantLinear | None" = None):
        """x_global_scale / return_output_scale chain quantized layers without a pass over the activation between them
        (single-GPU NVFP4 layers): with return_output_scale the GEMM's epilogue also forms the global scale of its
        output, and the call returns (y, y_global_scale); handing that to the next layer's forward as x_global_scale
        lets it quantize at once.  The bytes are those of the unchained layers."""
        if x_global_scale is not None or return_output_scale:
            return self._forward_chained(x, x_global_scale, return_output_scale, next_layer)
        if getattr(self, "_use_graph", False):
            return self._graphed_forward(x)
        return self._forward_impl(x)

    def _forward_chained(self, x, x_global_scale, return_output_scale, next_layer):
        if self.format != "nvfp4" or (self.parallel is not None and self.world > 1):
            raise ValueError("chained global scales are offered for single-GPU NVFP4 layers")
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1])
        if return_output_scale and not hasattr(self, "_out_scale_scratch"):
            self.register_buffer("_out_scale_scratch", torch.zeros(8, dtype=torch.int32, device=x2.device), persistent=False)
        res = ops.linear_forward_chained(
            x2, self.weight_fp4, self.weight_sf, self.weight_global_scale, self._scale_scratch, self.out_dtype,
            bias=self.bias.detach() if self.bias is not None else None, input_global_scale=x_global_scale,
            output_scale_scratch=self._out_scale_scratch if return_output_scale else None,
            next_weight_global_scale=next_layer.weight_global_scale if (return_output_scale and next_layer is not None) else None)
        if not return_output_scale:
            return res.reshape(*lead, res.shape[-1])
        y, y_gs, _ = res
        return y.reshape(*lead, y.shape[-1]), y_gs

    def _forward_impl(self, x: torch.Tensor) -> torch.Tensor:
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1])
        if self.parallel == "row" and not self.input_is_parallel:
            lo, hi = shard_range(self.in_features, self.rank, self.world, 4 * self.block, "in_features")
            x2 = x2[:, lo:hi]
        acc_dtype = torch.float32 if self.parallel == "row" and self.world > 1 else self.out_dtype
        if self.fused_gather and self.world > 1 and self.gather_output:
            return self._forward_fused_gather(x2, lead)
        if self.fused_reduce_scatter and self.world > 1 and x2.shape[0] % (32 * self.world) == 0:
            return self._forward_fused_reduce_scatter(x2)
        # the bias rides in the GEMM epilogue (added before the single rounding) wherever the local product is
        # already the final value of its columns; row-parallel partial sums get it after the reduction
        fused_bias = None
        if self.bias is not None and acc_dtype != torch.float32:
            fused_bias = self._bias_shard() if self.parallel == "column" and self.world > 1 else self.bias
            fused_bias = fused_bias.detach()
        if self.format == "nvfp4" and acc_dtype != torch.float32:
            # one extension call: global scale, alpha, quantize and GEMM (+ bias)
            y = ops.linear_forward(x2, self.weight_fp4, self.weight_sf, self.weight_global_scale, self._scale_scratch,
                                   acc_dtype, bias=fused_bias)
        elif self.format == "nvfp4":
            a_fp4, a_sf, alpha = self._quantize_activation(x2)
            y = ops.cutlass_scaled_fp4_mm(a_fp4, self.weight_fp4, a_sf, self._sf_view(self.weight_sf), alpha, acc_dtype,
                                          bias=fused_bias) \
                if acc_dtype != torch.float32 else self._mm_f32(a_fp4, a_sf, alpha)
        else:
            a_fp4, a_sf = ops.scaled_mxfp4_quant(x2, self.mx_rounding)
            y = ops.mxfp4_scaled_mm(a_fp4, self.weight_fp4, a_sf, self._sf_view(self.weight_sf), acc_dtype, bias=fused_bias) \
                if acc_dtype != torch.float32 else self._mm_f32(a_fp4, a_sf, None)
        y = self._combine(y)
        if self.bias is not None and fused_bias is None:
            y = y + (self.bias if y.shape[-1] == self.out_features else self._bias_shard())
        return y.reshape(*lead, y.shape[-1]) if y.shape[0] == x2.shape[0] else y

    def _forward_fused_gather(self, x2: torch.Tensor, lead) -> torch.Tensor:
        """Column-parallel forward whose result is the gathered [M, N] matrix; the returned tensor
        aliases a peer-visible buffer that the next call with the same M overwrites.  One extension call: quantizer
        and GEMM chained, the GEMM storing its tiles into every rank's buffer and synchronising the ranks itself
        (no barrier or collective around it)."""
        from ._ops_real import _load_scaled_fp4_ops
        from .peer import GatherBuffer
        m = x2.shape[0]
        gb = self._gather_buffers.get(m)
        if gb is None:
            gb = self._gather_buffers[m] = GatherBuffer(m, self.n_local, self.out_dtype, x2.device, self.process_group)
        gb.wait_limit_ns = self.peer_wait_limit_ns
        code = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}[self.out_dtype]
        if self.format == "nvfp4":
            ext = _load_scaled_fp4_ops(("linear_forward_gather", "linear_workspace_bytes"))
            if x2.stride(-1) != 1 or (m > 1 and x2.stride(0) % 8 != 0) or x2.data_ptr() % 16 != 0:
                x2 = x2.contiguous()
            workspace = torch.empty(ext.linear_workspace_bytes(m, x2.shape[1]), dtype=torch.uint8, device=x2.device)
            ext.linear_forward_gather(gb.dst_ptrs, gb.flag_ptrs, gb.rank, gb.wait_limit_ns, gb.ld, code, x2, self.weight_fp4,
                                      self.weight_sf, self.weight_global_scale, workspace, self._scale_scratch)
        else:
            ext = _load_scaled_fp4_ops(("scaled_fp4_mm_gather",))
            a_fp4, a_sf = ops.scaled_mxfp4_quant(x2, self.mx_rounding)
            ext.scaled_fp4_mm_gather(gb.dst_ptrs, gb.flag_ptrs, gb.rank, gb.wait_limit_ns, gb.ld, code, a_fp4, self.weight_fp4,
                                     a_sf.view(torch.uint8), self.weight_sf, None, True)
        y = gb.gathered()
        if self.bias is not None:
            y = y + self.bias
        return y.reshape(*lead, y.shape[-1])

    def forward_gather_fp4(self, x: torch.Tensor, out_global_scale: torch.Tensor):
        """Column-parallel NVFP4 layer whose gathered output is the next layer's NVFP4 activation operand: returns
        (packed uint8 [M, N / 2], float8_e4m3fn scales [round_up(M,128), N / 16]) of the whole [M, N] product, the
        bytes scaled_fp4_quant(layer(x), out_global_scale) would give, on every rank.  Each tile is quantized in the
        GEMM epilogue and 0.5625 bytes per element cross NVLink instead of 2.  `out_global_scale`: fp32 [1] on the
        device, the same (calibrated) value on every rank.  The result aliases a peer-visible buffer that the next
        call with the same M overwrites."""
        from ._ops_real import _load_scaled_fp4_ops
        from .peer import Fp4GatherBuffer
        assert self.parallel == "column" and self.format == "nvfp4", "column-parallel NVFP4 layers only"
        assert self.out_dtype in (torch.float16, torch.bfloat16)
        x2 = x.reshape(-1, x.shape[-1])
        m = x2.shape[0]
        if x2.stride(-1) != 1 or (m > 1 and x2.stride(0) % 8 != 0) or x2.data_ptr() % 16 != 0:
            x2 = x2.contiguous()
        key = ("fp4", m)
        gb = self._gather_buffers.get(key)
        if gb is None:
            gb = self._gather_buffers[key] = Fp4GatherBuffer(m, self.n_local, x2.device, self.process_group)
        gb.wait_limit_ns = self.peer_wait_limit_ns
        ext = _load_scaled_fp4_ops(("linear_forward_gather_fp4", "linear_workspace_bytes"))
        workspace = torch.empty(ext.linear_workspace_bytes(m, x2.shape[1]), dtype=torch.uint8, device=x2.device)
        bias = self._bias_shard().detach() if self.bias is not None and self.world > 1 else \
            (self.bias.detach() if self.bias is not None else None)
        ext.linear_forward_gather_fp4(gb.packed_ptrs, gb.sf_ptrs, gb.flag_ptrs, gb.rank, gb.wait_limit_ns, gb.n, gb.n_offset,
                                      1 if self.out_dtype == torch.bfloat16 else 0, x2, self.weight_fp4, self.weight_sf,
                                      self.weight_global_scale, bias, out_global_scale, workspace, self._scale_scratch)
        return gb.packed, gb.scales.view(torch.float8_e4m3fn)

    def _forward_fused_reduce_scatter(self, x2: torch.Tensor) -> torch.Tensor:
        """Row-parallel forward: returns this rank's [M / world, N] rows of the sum over ranks."""
        from ._ops_real import _load_scaled_fp4_ops
        from .peer import ReduceBuffer
        m = x2.shape[0]
        rb = self._reduce_buffers.get(m)
        if rb is None:
            rb = self._reduce_buffers[m] = ReduceBuffer(m, self.out_features, x2.device, self.process_group)
        rb.wait_limit_ns = self.peer_wait_limit_ns
        ext = _load_scaled_fp4_ops(("scaled_fp4_mm_reduce_scatter",))
        if self.format == "nvfp4":
            a_fp4, a_sf, alpha = self._quantize_activation(x2)
        else:
            a_fp4, a_sf = ops.scaled_mxfp4_quant(x2, self.mx_rounding)
            alpha = None
        # the kernel announces "ready" to the peers when it starts, i.e. after this zeroing in stream order, and
        # returns only when every rank's contributions have arrived
        rb.buf.zero_()
        ext.scaled_fp4_mm_reduce_scatter(rb.dst_ptrs, rb.flag_ptrs, rb.rank, rb.wait_limit_ns, a_fp4, self.weight_fp4,
                                         a_sf.view(torch.uint8), self.weight_sf, alpha, self.format == "mxfp4")
        y = rb.buf.to(self.out_dtype)
        if self.bias is not None:
            y = y + self.bias
        return y

    def _mm_f32(self, a_fp4, a_sf, alpha):
        """Unrounded fp32 partial product of a K-split layer (the public wrappers only offer fp16 / bf16 outputs,
        like the reference's); alpha is None for MXFP4."""
        from ._ops_real import _load_scaled_fp4_ops
        out = torch.empty((a_fp4.shape[0], self.weight_fp4.shape[0]), dtype=torch.float32, device=a_fp4.device)
        if self.format == "mxfp4":
            _load_scaled_fp4_ops(("mxfp4_scaled_mm",)).mxfp4_scaled_mm(
                out, a_fp4, self.weight_fp4, a_sf, self._sf_view(self.weight_sf), alpha)
        else:
            _load_scaled_fp4_ops(("cutlass_scaled_fp4_mm",)).cutlass_scaled_fp4_mm(
                out, a_fp4, self.weight_fp4, a_sf, self._sf_view(self.weight_sf), alpha)
        return out

    def _quantize_activation(self, x2: torch.Tensor):
        """(fp4, scales, alpha) of the NVFP4 activation.  One pass over x2 (global scale, alpha and quantization in
        one call) except for row-parallel layers, whose maximum needs an all-reduce between the two steps."""
        if self.parallel == "row" and self.world > 1:
            a_gs = self._activation_global_scale(x2)
            a_fp4, a_sf = ops.scaled_fp4_quant(x2, a_gs)
            return a_fp4, a_sf, ops.alpha_from_scales(a_gs, self.weight_global_scale)
        a_fp4, a_sf, _, alpha = ops.dynamic_scaled_fp4_quant(x2, self._scale_scratch, self.weight_global_scale)
        return a_fp4, a_sf, alpha

    def _activation_global_scale(self, x2: torch.Tensor) -> torch.Tensor:
        if self.parallel == "row" and self.world > 1:
            # every rank must quantize its K-slice with the scale of the WHOLE activation:
            # max-reduce the per-rank amax bit patterns (non-negative floats order like ints)
            import torch.distributed as dist
            scratch = torch.empty(2, dtype=torch.int32, device=x2.device)
            ops.global_scale(x2, scratch)
            bits = scratch[:1]                       # word 0: fp32 bit pattern of this rank's amax
            dist.all_reduce(bits, op=dist.ReduceOp.MAX, group=self.process_group)
            amax = bits.view(torch.float32)
            amax = torch.where(amax == 0, torch.ones_like(amax), amax)
            return (448.0 * 6.0) / amax
        return ops.global_scale(x2)

    def _combine(self, y: torch.Tensor) -> torch.Tensor:
        if self.world == 1 or self.parallel is None:
            return y
        import torch.distributed as dist
        if self.parallel == "column":
            if not self.gather_output:
                return y
            parts = torch.empty((self.world * y.shape[0], y.shape[1]), dtype=y.dtype, device=y.device)
            dist.all_gather_into_tensor(parts, y.contiguous(), group=self.process_group)
            return gather_columns_layout(parts.view(self.world, *y.shape))
        # row-parallel: fp32 partial sums, reduce-scatter over rows, round once
        m = y.shape[0]
        if m % self.world != 0:
            dist.all_reduce(y, group=self.process_group)
            return y.to(self.out_dtype)
        out = torch.empty((m // self.world, y.shape[1]), dtype=y.dtype, device=y.device)
        dist.reduce_scatter_tensor(out, y.contiguous(), group=self.process_group)
        return out.to(self.out_dtype)

    def _bias_shard(self):
        lo, hi = shard_range(self.out_features, self.rank, self.world, 128, "out_features")
        return self.bias[lo:hi]

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, format={self.format}, "
                f"parallel={self.parallel}, world={self.world}")
