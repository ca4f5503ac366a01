"""Import-name compatibility: `import nvfp` / `import nvfp.ops` resolve to the
B200-native package, as scripts written against huweim/nvfp_kernel expect."""
from nvfp_kernel_b200 import *  # noqa: F401,F403
from nvfp_kernel_b200 import __all__  # noqa: F401
