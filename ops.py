"""Re-export of the op API for scripts that ``import ops`` from the repository root, as the
reference's scripts do (speed_test.py:5 there; same shim as its ops.py:2-7)."""
from nvfp_kernel_b200.ops import (  # noqa: F401
    cutlass_scaled_fp4_mm,
    get_active_backend,
    reciprocal_approximate_ftz_tensor,
    scaled_fp4_quant,
)
