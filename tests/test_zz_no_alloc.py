"""nvfp_global_scale_noalloc: the global scale for callers that cannot allocate scratch
(their device allocator is frozen, or cudaMalloc is off limits on their threads).  The amax
word sits in a static device array inside the library, shared by all calls, so the test makes
two calls in a row -- the second on data with a SMALLER maximum, which only passes if the
call clears what the first one left behind -- and compares each with nvfp_global_scale
(caller-provided scratch), bit for bit.  Collected last on purpose (file name)."""
import pytest
import torch

from helpers import capi_global_scale
from inputs import make_input
from nvfp_kernel_b200 import _capi

pytestmark = pytest.mark.gpu


def _noalloc(x: torch.Tensor) -> torch.Tensor:
    lib = _capi.load()
    gs = torch.empty(1, dtype=torch.float32, device=x.device)
    m, n = x.shape
    dt = _capi.NVFP_DTYPE_BF16 if x.dtype == torch.bfloat16 else _capi.NVFP_DTYPE_F16
    _capi.check(lib.nvfp_global_scale_noalloc(gs.data_ptr(), x.data_ptr(), m, n, x.stride(0) if m > 1 else n, dt,
                                              torch.cuda.current_stream().cuda_stream))
    return gs


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_two_calls_in_a_row_match_the_scratch_taking_entry_point(dtype):
    big = (make_input("large", (513, 1024), dtype, seed=1)).cuda()        # amax in the hundreds
    small = (make_input("small", (129, 80), dtype, seed=2)).cuda()        # amax ~ 0.004
    for x in (big, small, big):
        got, want = _noalloc(x), capi_global_scale(x)
        assert got.item() == want.item(), (tuple(x.shape), got.item(), want.item())
    zero = torch.zeros((4, 64), dtype=dtype, device="cuda")
    assert _noalloc(zero).item() == 2688.0


def test_rejects_tensors_beyond_the_stated_maximum():
    lib = _capi.load()
    x = torch.zeros((8, 64), dtype=torch.bfloat16, device="cuda")
    gs = torch.empty(1, dtype=torch.float32, device="cuda")
    rc = lib.nvfp_global_scale_noalloc(gs.data_ptr(), x.data_ptr(), 1 << 20, 1 << 13, 1 << 13,
                                       _capi.NVFP_DTYPE_BF16, None)
    assert rc == _capi.NVFP_ERR_INVALID_ARGUMENT and b"at most" in lib.nvfp_last_error()
