"""QuantLinear(mode="real") end to end on one GPU."""
import pytest
import torch

from inputs import gemm_inputs

pytestmark = pytest.mark.gpu


def _reference_flow(a, w):
    """The reference's FP4GemmWithOnlineActivation (speed_test.py:36-50) written with the
    public ops of this package."""
    import nvfp.ops as ops
    w_amax = torch.abs(w).max().to(torch.float32)
    w_scale = 2688.0 / w_amax
    w_fp4, s_w = ops.scaled_fp4_quant(w, w_scale.reshape(1))
    a_amax = torch.abs(a).max().to(torch.float32)
    a_scale = 2688.0 / a_amax
    a_fp4, s_a = ops.scaled_fp4_quant(a, a_scale.reshape(1))
    alpha = 1.0 / (a_scale * w_scale)
    return ops.cutlass_scaled_fp4_mm(a_fp4, w_fp4, s_a, s_w, alpha.reshape(1), torch.bfloat16)


@pytest.mark.parametrize("m,n,k", [(4, 256, 512), (130, 384, 1024), (1024, 1024, 1024)])
def test_quant_linear_equals_reference_flow(m, n, k):
    from nvfp_kernel_b200 import QuantLinear
    a, w = gemm_inputs(m, n, k, seed=1, w_std=0.05)
    a, w = a.cuda(), w.cuda()
    lin = torch.nn.Linear(k, n, bias=True, device="cuda", dtype=torch.bfloat16)
    lin.weight.data.copy_(w)
    q = QuantLinear.from_linear(lin)
    y = q(a)
    # without the bias: exactly the reference's flow
    product = _reference_flow(a, w)
    q_nobias = QuantLinear(k, n, device="cuda").load_weight(w)
    assert torch.equal(q_nobias(a), product)
    # the bias is added in the GEMM epilogue before the one rounding to bf16, so the result is at least as close
    # to product + bias as adding it to the rounded product would be
    want = product.float() + lin.bias.float()
    # (half a bf16 ulp, 2^-8 relative, for the rounding of `product` plus the same for the rounding of y)
    assert ((y.float() - want).abs() <= 2.0 ** -7 * (product.float().abs() + lin.bias.float().abs()) + 1e-6).all()
    dense = lin(a)
    assert (y.float() - dense.float()).abs().max() < 0.3 * dense.float().abs().max()
    # leading dims are preserved
    y3 = q(a.reshape(2, m // 2, k))
    assert y3.shape == (2, m // 2, n) and torch.equal(y3.reshape(m, n), y)
    # state round trip without re-quantizing
    q2 = QuantLinear(k, n, bias=True, device="cuda")
    q2.load_state_dict(q.state_dict())
    assert torch.equal(q2(a), y)


def test_quant_linear_mxfp4():
    from nvfp_kernel_b200 import QuantLinear
    a, w = gemm_inputs(96, 256, 512, seed=2, w_std=0.02)
    a, w = a.cuda(), w.cuda()
    q = QuantLinear(512, 256, format="mxfp4", device="cuda").load_weight(w)
    y = q(a)
    dense = a.float() @ w.float().T
    assert y.dtype == torch.bfloat16 and (y.float() - dense).abs().max() < 0.3 * dense.abs().max()


def test_cuda_graph_replay_matches_eager_and_handles_several_shapes():
    from nvfp_kernel_b200 import QuantLinear
    a, w = gemm_inputs(16, 512, 1024, seed=5, w_std=0.05)
    a, w = a.cuda(), w.cuda()
    eager = QuantLinear(1024, 512, device="cuda").load_weight(w)
    graphed = QuantLinear(1024, 512, device="cuda").load_weight(w).enable_cuda_graph()
    for scale in (1.0, 0.3, 7.0):                       # replays must pick up new input values
        assert torch.equal(graphed(a * scale), eager(a * scale))
    b = (a[:4] * 2).contiguous()                        # a second shape gets its own graph
    assert torch.equal(graphed(b), eager(b))
    assert torch.equal(graphed(a), eager(a))
    # writing into the graph's own input buffer and passing it saves the copy
    buf = graphed.graph_input((16, 1024), torch.bfloat16)
    buf.copy_(a * 0.5)
    assert torch.equal(graphed(buf), eager(a * 0.5))
    fresh = QuantLinear(1024, 512, device="cuda").load_weight(w).enable_cuda_graph()
    buf2 = fresh.graph_input((16, 1024))                # captured before any forward, on an all-zero activation
    buf2.copy_(a)
    assert torch.equal(fresh(buf2), eager(a))
    import nvfp_kernel_b200 as nv
    assert nv.device_status() == 0


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
def test_quantize_linear_layers_of_a_model(dt):
    import torch.nn as nn
    from nvfp_kernel_b200 import QuantLinear
    from nvfp_kernel_b200.convert import quantize_linear_layers
    torch.manual_seed(0)
    model = nn.Sequential()
    model.add_module("up", nn.Linear(256, 512, bias=False))
    model.add_module("act", nn.SiLU())
    model.add_module("down", nn.Linear(512, 256, bias=True))
    model.add_module("lm_head", nn.Linear(256, 96, bias=False))
    model = model.cuda().to(dt)
    x = torch.randn(40, 256, device="cuda", dtype=dt)
    dense = model(x)
    names = quantize_linear_layers(model)
    assert names == ["up", "down"] and isinstance(model.up, QuantLinear) and isinstance(model.lm_head, nn.Linear)
    # the replaced layers keep the model's dtype (an fp16 model must not turn bf16 half-way through)
    assert model.up.out_dtype == dt and model.down.bias.dtype == dt
    y = model(x)
    assert y.shape == dense.shape and y.dtype == dt
    assert (y.float() - dense.float()).abs().max() < 0.35 * dense.float().abs().max()


def test_host_pipeline_matches_direct_calls():
    """Calls on pinned host buffers with copy-in, compute and copy-out of consecutive calls overlapped: every
    result equals layer(x.cuda()).cpu() bit for bit, also when shapes change between calls and when the layer
    hands back one reused output buffer."""
    import nvfp_kernel_b200 as nv
    from nvfp_kernel_b200 import HostPipeline, QuantLinear
    torch.manual_seed(3)
    layer = QuantLinear(512, 384, device="cuda").load_weight((torch.randn(384, 512) * 0.05).to(torch.bfloat16).cuda())
    xs = [(torch.randn(m, 512) * (1 + i)).to(torch.bfloat16).pin_memory() for i, m in enumerate((256, 256, 256, 64, 256, 1))]
    outs = [torch.empty((x.shape[0], 384), dtype=torch.bfloat16).pin_memory() for x in xs]
    pipe = HostPipeline(layer, depth=2)
    for x, o in zip(xs, outs):
        pipe.submit(x, o)
    pipe.synchronize()
    for x, o in zip(xs, outs):
        assert torch.equal(o, layer(x.cuda()).cpu())
    static_out = torch.empty((256, 384), dtype=torch.bfloat16, device="cuda")

    def reusing(x):
        static_out.copy_(layer(x))
        return static_out

    pipe = HostPipeline(reusing, depth=2, device="cuda", reuses_output=True)
    outs2 = [torch.empty((256, 384), dtype=torch.bfloat16).pin_memory() for _ in range(3)]
    for x, o in zip(xs[:3], outs2):
        pipe.submit(x, o)
    pipe.synchronize()
    for x, o in zip(xs[:3], outs2):
        assert torch.equal(o, layer(x.cuda()).cpu())
    assert nv.device_status() == 0


@pytest.mark.parametrize("m,n,k", [(1, 4096, 4096), (16, 6144, 4096), (8, 4096, 14336), (48, 256, 1024), (128, 512, 2048),
                                   (300, 384, 1024), (2048, 4096, 4096), (1024, 8192, 1024), (2048, 4096, 2048),
                                   (100, 1024, 8192)])
def test_one_call_forward_equals_the_separate_calls(m, n, k):
    """nvfp_linear_forward (quantizer and GEMM issued by one call; while the quantizer is the one-pass kernel the
    GEMM -- few-rows, 128-row-tile or CTA-pair kernel -- is launched under it and fetches its weights meanwhile) gives
    the bytes of nvfp_dynamic_fp4_quant + nvfp_scaled_fp4_mm(_bias), call after call with changing inputs, with and
    without a bias."""
    from helpers import capi_dynamic_quant, capi_global_scale, capi_linear_forward, capi_mm, capi_quant
    a, w = gemm_inputs(m, n, k, seed=m + n + k, w_std=0.05)
    a, w = a.cuda(), w.cuda()
    w_gs = capi_global_scale(w)
    w_fp4, w_sf = capi_quant(w, w_gs)
    scratch = torch.zeros(8, dtype=torch.int32, device="cuda")
    bias = (torch.randn(n) * 0.1).to(torch.bfloat16).cuda()
    for i in range(4):
        x = (a * (1.0 + 0.5 * i)).to(torch.bfloat16)
        b = bias if i % 2 else None
        got = capi_linear_forward(x, w_fp4, w_sf, w_gs, scratch, torch.bfloat16, b)
        a_fp4, a_sf, _, alpha = capi_dynamic_quant(x, scratch, w_gs)
        want = capi_mm(a_fp4, w_fp4, a_sf, w_sf, alpha, torch.bfloat16, bias=b)
        assert torch.equal(got, want), (i, m, n, k)


def test_two_layers_chained_through_nvfp4_output():
    """Layer 1 writes its result as NVFP4 straight from the GEMM epilogue (calibrated output scale), layer 2
    consumes it: bit-identical to layer 1 -> bf16 tensor -> quantizer -> layer 2, with one kernel and one
    [m, n] round trip through memory fewer."""
    import nvfp_kernel_b200 as nv
    torch.manual_seed(11)
    m, k, n1, n2 = 512, 1024, 4096, 512
    x = torch.randn(m, k).to(torch.bfloat16).cuda()
    w1 = (torch.randn(n1, k) * 0.05).to(torch.bfloat16).cuda()
    w2 = (torch.randn(n2, n1) * 0.02).to(torch.bfloat16).cuda()
    gx, g1, g2 = nv.global_scale(x), nv.global_scale(w1), nv.global_scale(w2)
    x_fp4, x_sf = nv.scaled_fp4_quant(x, gx)
    w1_fp4, w1_sf = nv.scaled_fp4_quant(w1, g1)
    w2_fp4, w2_sf = nv.scaled_fp4_quant(w2, g2)
    alpha1 = nv.alpha_from_scales(gx, g1)
    # unfused chain; its hidden tensor also provides the "calibrated" scale of the hidden activation
    h = nv.cutlass_scaled_fp4_mm(x_fp4, w1_fp4, x_sf, w1_sf, alpha1, torch.bfloat16)
    gh = nv.global_scale(h)
    h_fp4, h_sf = nv.scaled_fp4_quant(h, gh)
    alpha2 = nv.alpha_from_scales(gh, g2)
    want = nv.cutlass_scaled_fp4_mm(h_fp4, w2_fp4, h_sf, w2_sf, alpha2, torch.bfloat16)
    # fused: no hidden bf16 tensor
    f_fp4, f_sf = nv.scaled_fp4_mm_fp4out(x_fp4, w1_fp4, x_sf, w1_sf, alpha1, gh, torch.bfloat16)
    assert torch.equal(f_fp4, h_fp4) and torch.equal(f_sf.view(torch.uint8), h_sf.view(torch.uint8))
    got = nv.cutlass_scaled_fp4_mm(f_fp4, w2_fp4, f_sf, w2_sf, alpha2, torch.bfloat16)
    assert torch.equal(got, want)
    assert nv.device_status() == 0


@pytest.mark.parametrize("m,k,inter,hidden", [(300, 1024, 1440, 512), (2048, 1024, 2048, 1024), (40, 512, 256, 256),
                                              (1, 4096, 1024, 512), (16, 8192, 2048, 256), (40, 512, 1440, 512),
                                              (100, 2048, 1440, 256), (128, 1024, 4096, 128), (16, 1024, 12288, 256), (7, 512, 9536, 128)])
def test_gated_mlp_with_activation_and_quantizer_in_the_epilogue(m, k, inter, hidden):
    """x -> gate/up GEMM with silu(gate)*up (and the NVFP4 quantization of the result) in its epilogue -> down GEMM,
    against the same chain with the bf16 gate/up product, torch's silu * mul and the quantizer kernel in between."""
    import torch.nn.functional as F
    import nvfp_kernel_b200 as nv
    torch.manual_seed(m + inter)
    x = torch.randn(m, k).to(torch.bfloat16).cuda()
    w_gate = (torch.randn(inter, k) * 0.05).to(torch.bfloat16).cuda()
    w_up = (torch.randn(inter, k) * 0.05).to(torch.bfloat16).cuda()
    w_down = (torch.randn(hidden, inter) * 0.03).to(torch.bfloat16).cuda()
    w_gu = nv.interleave_gate_up(w_gate, w_up)
    assert torch.equal(w_gu.view(inter // 16, 2, 16, k)[:, 0].reshape(inter, k), w_gate)
    gx, ggu, gd = nv.global_scale(x), nv.global_scale(w_gu), nv.global_scale(w_down)
    x_fp4, x_sf = nv.scaled_fp4_quant(x, gx)
    gu_fp4, gu_sf = nv.scaled_fp4_quant(w_gu, ggu)
    d_fp4, d_sf = nv.scaled_fp4_quant(w_down, gd)
    alpha1 = nv.alpha_from_scales(gx, ggu)
    # separate kernels
    y = nv.cutlass_scaled_fp4_mm(x_fp4, gu_fp4, x_sf, gu_sf, alpha1, torch.bfloat16).view(m, inter // 16, 2, 16)
    h = F.silu(y[:, :, 0].reshape(m, inter)) * y[:, :, 1].reshape(m, inter)
    # activation in the epilogue, bf16 out: torch's result up to the last bit of its exp
    h_f = nv.scaled_fp4_mm_silu_mul(x_fp4, gu_fp4, x_sf, gu_sf, alpha1, torch.bfloat16)
    assert h_f.shape == (m, inter)
    diff = (h_f.float() - h.float()).abs()
    assert (diff <= 2.0 ** -7 * h.float().abs() + 1e-30).all()
    assert (h_f == h).float().mean() > 0.999
    # activation and quantizer in the epilogue: exactly the quantizer's bytes for that activation
    gh = nv.global_scale(h_f)
    want_fp4, want_sf = nv.scaled_fp4_quant(h_f, gh)
    got_fp4, got_sf = nv.scaled_fp4_mm_silu_mul(x_fp4, gu_fp4, x_sf, gu_sf, alpha1, torch.bfloat16, out_global_scale=gh)
    assert torch.equal(got_fp4, want_fp4) and torch.equal(got_sf.view(torch.uint8), want_sf.view(torch.uint8))
    alpha2 = nv.alpha_from_scales(gh, gd)
    out = nv.cutlass_scaled_fp4_mm(got_fp4, d_fp4, got_sf, d_sf, alpha2, torch.bfloat16)
    assert torch.equal(out, nv.cutlass_scaled_fp4_mm(want_fp4, d_fp4, want_sf, d_sf, alpha2, torch.bfloat16))
    dense = F.linear(F.silu(F.linear(x, w_gate)) * F.linear(x, w_up), w_down)
    assert (out.float() - dense.float()).abs().max() < 0.35 * dense.float().abs().max()
    assert nv.device_status() == 0


@pytest.mark.parametrize("m,hidden,inter", [(1, 4096, 1024), (16, 1024, 12288), (40, 512, 1440), (128, 1024, 4096),
                                            (300, 1024, 1440), (2048, 1024, 2048), (5000, 512, 512)])
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
def test_one_call_gated_mlp_equals_the_separate_calls(m, hidden, inter, dt):
    """nvfp_gated_mlp_forward (quantizer, gate/up GEMM and down GEMM chained with programmatic dependent launch, each
    GEMM fetching its weights while the kernel before it still runs) against the same three steps as separate calls:
    identical bytes, on shapes that take each of the three GEMM kernels, the one-pass and the two-launch quantizer,
    called twice in a row so that a call's first kernel follows the previous call's last."""
    from helpers import capi_gated_mlp_forward
    import nvfp_kernel_b200 as nv
    torch.manual_seed(m + inter)
    x = torch.randn(m, hidden).to(dt).cuda()
    w_gu = nv.interleave_gate_up((torch.randn(inter, hidden) * 0.05).to(dt).cuda(), (torch.randn(inter, hidden) * 0.05).to(dt).cuda())
    w_d = (torch.randn(hidden, inter) * 0.03).to(dt).cuda()
    ggu, gd = nv.global_scale(w_gu), nv.global_scale(w_d)
    gu_fp4, gu_sf = nv.scaled_fp4_quant(w_gu, ggu)
    d_fp4, d_sf = nv.scaled_fp4_quant(w_d, gd)
    scratch = torch.zeros(8, dtype=torch.int32, device="cuda")
    x_fp4, x_sf, _, alpha1 = nv.dynamic_scaled_fp4_quant(x, scratch, ggu)
    gh = nv.global_scale(nv.scaled_fp4_mm_silu_mul(x_fp4, gu_fp4, x_sf, gu_sf, alpha1, dt))
    alpha2 = nv.alpha_from_scales(gh, gd)
    h_fp4, h_sf = nv.scaled_fp4_mm_silu_mul(x_fp4, gu_fp4, x_sf, gu_sf, alpha1, dt, out_global_scale=gh)
    want = nv.cutlass_scaled_fp4_mm(h_fp4, d_fp4, h_sf, d_sf, alpha2, dt)
    for _ in range(2):
        got = capi_gated_mlp_forward(x, gu_fp4, gu_sf, ggu, d_fp4, d_sf, gh, alpha2, scratch, dt)
        assert torch.equal(got, want)
    assert torch.equal(nv.gated_mlp_forward(x, gu_fp4, gu_sf, ggu, d_fp4, d_sf, gh, alpha2, scratch, dt), want)


def test_quant_gated_mlp_module():
    """QuantGatedMLP (three launches, calibrated hidden scale) against its own separate-kernel path (dynamic hidden
    scale): with the scale calibrated on the very input both quantize the hidden activation with the same scale, so
    the outputs are identical; on other inputs they stay close; state round trip; result near the dense MLP."""
    from nvfp_kernel_b200 import QuantGatedMLP
    from nvfp_kernel_b200.mlp import dense_gated_mlp
    torch.manual_seed(2)
    hidden, inter, m = 512, 1408, 192
    x = torch.randn(m, hidden).to(torch.bfloat16).cuda()
    wg = (torch.randn(inter, hidden) * 0.05).to(torch.bfloat16).cuda()
    wu = (torch.randn(inter, hidden) * 0.05).to(torch.bfloat16).cuda()
    wd = (torch.randn(hidden, inter) * 0.03).to(torch.bfloat16).cuda()
    mlp = QuantGatedMLP(hidden, inter, device="cuda").load_weights(wg, wu, wd).calibrate(x)
    y = mlp(x)
    assert y.shape == (m, hidden) and y.dtype == torch.bfloat16
    assert torch.equal(y, mlp.reference_forward(x))
    x2 = (x * 0.7).to(torch.bfloat16)
    y2, ref2 = mlp(x2.reshape(2, m // 2, hidden)), mlp.reference_forward(x2)
    assert y2.shape == (2, m // 2, hidden)
    assert (y2.reshape(m, hidden).float() - ref2.float()).abs().max() <= 0.08 * ref2.float().abs().max()
    dense = dense_gated_mlp(x, wg, wu, wd)
    assert (y.float() - dense.float()).abs().max() < 0.35 * dense.float().abs().max()
    clone = QuantGatedMLP(hidden, inter, device="cuda")
    clone.load_state_dict(mlp.state_dict())
    assert torch.equal(clone(x), y)
    import nvfp_kernel_b200 as nv
    assert nv.device_status() == 0


def test_model_surgery_replaces_gated_mlp_blocks():
    """quantize_gated_mlps on a toy Llama-style model: the gate/up/down blocks with a SiLU become QuantGatedMLP with
    scales calibrated by a run of the unquantized model, other blocks stay, and the model's output stays close."""
    import torch.nn as nn
    from nvfp_kernel_b200 import QuantGatedMLP
    from nvfp_kernel_b200.convert import quantize_gated_mlps

    class MLP(nn.Module):
        def __init__(self, hidden, inter, act):
            super().__init__()
            self.gate_proj = nn.Linear(hidden, inter, bias=False)
            self.up_proj = nn.Linear(hidden, inter, bias=False)
            self.down_proj = nn.Linear(inter, hidden, bias=False)
            self.act_fn = act

        def forward(self, x):
            return self.down_proj(self.act_fn(self.gate_proj(x)) * self.up_proj(x))

    class Block(nn.Module):
        def __init__(self, hidden, inter, act):
            super().__init__()
            self.norm = nn.LayerNorm(hidden)
            self.mlp = MLP(hidden, inter, act)

        def forward(self, x):
            return x + self.mlp(self.norm(x))

    torch.manual_seed(3)
    hidden, inter = 256, 704
    model = nn.Sequential(Block(hidden, inter, nn.SiLU()), Block(hidden, inter, nn.SiLU()), Block(hidden, inter, nn.GELU()))
    model = model.to(torch.bfloat16).cuda()
    x = torch.randn(48, hidden).to(torch.bfloat16).cuda()
    with torch.no_grad():
        want = model(x)
    replaced = quantize_gated_mlps(model, lambda: model(x))
    assert replaced == ["0.mlp", "1.mlp"]
    assert isinstance(model[0].mlp, QuantGatedMLP) and isinstance(model[1].mlp, QuantGatedMLP)
    assert not isinstance(model[2].mlp, QuantGatedMLP)            # GELU: left alone
    assert float(model[0].mlp.act_global_scale) != float(model[1].mlp.act_global_scale)
    with torch.no_grad():
        got = model(x)
    assert got.shape == want.shape
    assert (got.float() - want.float()).abs().max() < 0.2 * want.float().abs().max()
    import nvfp_kernel_b200 as nv
    assert nv.device_status() == 0


def test_llama_model_from_transformers_with_quantized_layers():
    """A small random-initialised LlamaForCausalLM: attention projections swapped by quantize_linear_layers, MLP blocks
    by quantize_gated_mlps; the logits stay aligned with the unquantized model's (the reference's own model-level
    check is a llama-2-7b generation log, tmp.log:1-7 there; weights cannot be downloaded here)."""
    transformers = pytest.importorskip("transformers")
    from nvfp_kernel_b200 import QuantGatedMLP, QuantLinear
    from nvfp_kernel_b200.convert import quantize_gated_mlps, quantize_linear_layers
    torch.manual_seed(11)
    cfg = transformers.LlamaConfig(hidden_size=256, intermediate_size=704, num_hidden_layers=2, num_attention_heads=4,
                                   num_key_value_heads=4, vocab_size=512, max_position_embeddings=128)
    model = transformers.LlamaForCausalLM(cfg).to(torch.bfloat16).cuda().eval()
    ids = torch.randint(0, 512, (2, 24), device="cuda")
    with torch.no_grad():
        want = model(ids).logits.float()
    mlps = quantize_gated_mlps(model, lambda: model(ids))
    linears = quantize_linear_layers(model)
    assert len(mlps) == 2 and all(isinstance(layer.mlp, QuantGatedMLP) for layer in model.model.layers)
    assert len(linears) == 8 and isinstance(model.model.layers[0].self_attn.q_proj, QuantLinear)
    assert isinstance(model.lm_head, torch.nn.Linear)
    with torch.no_grad():
        got = model(ids).logits.float()
    cos = torch.nn.functional.cosine_similarity(got.flatten(), want.flatten(), dim=0).item()
    assert cos > 0.94, cos        # 4-bit operands in all ten GEMMs of a random-initialised model: 0.96 measured
    import nvfp_kernel_b200 as nv
    assert nv.device_status() == 0


def test_empty_batches():
    """Zero rows (an empty batch) and zero output columns go through every entry point without a launch that
    touches memory: empty results of the right shape, 2688 as the global scale of an empty activation."""
    import nvfp_kernel_b200 as nv
    from nvfp_kernel_b200 import QuantLinear
    from helpers import capi_dynamic_quant, capi_linear_forward, capi_mm, capi_quant
    w = (torch.randn(256, 512) * 0.05).to(torch.bfloat16).cuda()
    layer = QuantLinear(512, 256, bias=True, device="cuda").load_weight(w)
    x0 = torch.empty((0, 512), dtype=torch.bfloat16, device="cuda")
    y0 = layer(x0)
    assert y0.shape == (0, 256) and y0.dtype == torch.bfloat16
    assert layer(x0.reshape(0, 4, 512)).shape == (0, 4, 256)
    scratch = torch.zeros(8, dtype=torch.int32, device="cuda")
    fp4, sf, gs, _ = capi_dynamic_quant(x0, scratch, None)
    assert fp4.shape == (0, 256) and sf.shape == (0, 32) and gs.item() == 2688.0
    fp4, sf = capi_quant(x0, gs)
    assert fp4.numel() == 0 and sf.numel() == 0
    out = capi_mm(fp4, layer.weight_fp4, sf, layer.weight_sf, torch.ones(1, device="cuda"), torch.bfloat16)
    assert out.shape == (0, 256)
    out = capi_linear_forward(x0, layer.weight_fp4, layer.weight_sf, layer.weight_global_scale, scratch)
    assert out.shape == (0, 256)
    # the layer still works afterwards (scratch state intact)
    x = torch.randn(8, 512).to(torch.bfloat16).cuda()
    ref = QuantLinear(512, 256, bias=True, device="cuda").load_weight(w)
    assert torch.equal(layer(x), ref(x))
    assert nv.device_status() == 0


def test_speed_test_tables_run(capsys):
    """The timing tables of the package (the counterpart of the reference's speed_test.py) still run end to end."""
    from nvfp_kernel_b200 import speed_test
    speed_test.decode(1)
    speed_test.quant(1)
    out = capsys.readouterr().out
    assert out.count("\n") >= 12 + 5 + 4 and "14336" in out and "28672" in out


# shapes that take the CTA-pair kernel, the one-CTA tile kernel and the few-rows kernel
@pytest.mark.parametrize("m,k,n1,n2", [(2048, 1024, 2048, 1024), (300, 512, 1024, 512), (100, 512, 384, 256), (16, 1024, 4096, 1024),
                                       (1, 4096, 4096, 4096), (4096, 2048, 4096, 2048)])
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
def test_global_scale_from_the_producers_epilogue_chains_two_layers(m, k, n1, n2, dt):
    """Layer 1's GEMM forms the global scale of its output in its epilogue; layer 2 quantizes with it at once.  The
    scale equals nvfp_global_scale of layer 1's output bit for bit, and layer 2's result equals the unchained layer's
    (GEMM -> global scale -> quantizer -> GEMM), also with a bias in layer 1 and on repeated calls."""
    import nvfp_kernel_b200 as nv
    from helpers import capi_global_scale
    torch.manual_seed(m + n1)
    x = torch.randn(m, k).to(dt).cuda()
    l1 = nv.QuantLinear(k, n1, bias=True, out_dtype=dt, device="cuda").load_weight((torch.randn(n1, k) * 0.05).to(dt).cuda())
    l1.bias.data.copy_((torch.randn(n1) * 0.5).to(dt))
    l2 = nv.QuantLinear(n1, n2, out_dtype=dt, device="cuda").load_weight((torch.randn(n2, n1) * 0.05).to(dt).cuda())
    for scale in (1.0, 0.125, 3.0):                 # the scratch cleans itself between calls
        xs = (x * scale).to(dt)
        y_plain = l1(xs)
        z_plain = l2(y_plain)
        y, y_gs = l1(xs, return_output_scale=True, next_layer=l2)
        assert torch.equal(y, y_plain)
        assert torch.equal(y_gs, capi_global_scale(y_plain)), (y_gs.item(), capi_global_scale(y_plain).item())
        z = l2(y, x_global_scale=y_gs)
        assert torch.equal(z, z_plain)
    # both ends open at once: a middle layer takes a known scale and hands on its own
    z2, z2_gs = l2(y, x_global_scale=y_gs, return_output_scale=True)
    assert torch.equal(z2, z_plain) and torch.equal(z2_gs, capi_global_scale(z_plain))
    # a NaN in layer 1's output (here through its bias) makes the scale NaN, as 2688 / torch.abs(y).max() would be; an
    # infinity makes it 0; the scratch serves a clean call afterwards
    good = l1.bias.data.clone()
    for special in (float("nan"), float("inf")):
        l1.bias.data[n1 // 2] = special
        y_bad, gs_bad = l1(x, return_output_scale=True, next_layer=l2)
        want = (448.0 * 6.0) / torch.abs(y_bad).max().to(torch.float32)
        assert (torch.isnan(gs_bad).all() and torch.isnan(want)) if special != special else gs_bad.item() == want.item() == 0.0
        l1.bias.data.copy_(good)
    y, y_gs = l1(x, return_output_scale=True, next_layer=l2)
    assert torch.equal(y_gs, capi_global_scale(l1(x)))
    assert nv.device_status() == 0


def test_empty_batches():
    """Zero rows: every level returns empty results of the right shape and launches nothing that could fault; a batch
    of ordinary size right after is unaffected."""
    import nvfp_kernel_b200 as nv
    from helpers import capi_dynamic_quant, capi_global_scale, capi_mm, capi_quant
    k, n = 256, 384
    w = (torch.randn(n, k) * 0.05).to(torch.bfloat16).cuda()
    layer = nv.QuantLinear(k, n, bias=True, device="cuda").load_weight(w)
    empty = torch.empty((0, k), dtype=torch.bfloat16, device="cuda")
    y = layer(empty)
    assert y.shape == (0, n) and y.dtype == torch.bfloat16
    q, sf = nv.scaled_fp4_quant(empty, torch.ones(1, device="cuda"))
    assert q.shape == (0, k // 2) and sf.shape[0] == 0
    # the C ABI with m == 0: nothing written, status OK
    one = torch.ones(1, device="cuda")
    cq, csf = capi_quant(empty, one)
    assert cq.numel() == 0 and csf.numel() == 0
    w_gs = capi_global_scale(w)
    w4, wsf = capi_quant(w, w_gs)
    out = capi_mm(cq, w4, csf, wsf, one, torch.bfloat16)
    assert out.shape == (0, n)
    scratch = torch.zeros(8, dtype=torch.int32, device="cuda")
    dq = capi_dynamic_quant(empty, scratch, w_gs)
    assert dq[0].numel() == 0
    x = torch.randn(64, k).to(torch.bfloat16).cuda()
    assert torch.equal(layer(x), layer(x.clone())) and nv.device_status() == 0
