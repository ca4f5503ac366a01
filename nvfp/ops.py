from nvfp_kernel_b200.ops import *  # noqa: F401,F403
from nvfp_kernel_b200.ops import (  # noqa: F401
    cutlass_scaled_fp4_mm, get_active_backend, reciprocal_approximate_ftz_tensor, scaled_fp4_quant)
