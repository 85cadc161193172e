"""B200-native SSPA packed-KV decode path (sm_100a CUDA behind a C ABI).

Drop-in for the packed/active cache API of ``r2omni.sspa`` (R2-Omni):
``build_three_precision_cache``, ``ThreePrecisionCache``, ``allocate_splitk_workspace``,
``prepare_splitk_executor``, ``SplitKExecutor``, ``stack_homogeneous_splitk_executors``,
``append_generated_token``, ``append_recent_fp_triton`` -- same names, argument
meaning and error behaviour, hand-written CUDA underneath.  There is no CPU or
Triton fallback: importing the compute entry points without the built shared
library raises.
"""
from .sspa import *  # noqa: F401,F403
from .sspa import __all__  # noqa: F401
