"""QuantLinear(mode="real") end to end on one GPU."""
import pytest
import torch

from helpers import check_gemm
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
    want = _reference_flow(a, w) + lin.bias
    assert torch.equal(y, want)
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
