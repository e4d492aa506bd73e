"""Same shim as the reference's fasteq/ops/so3_linear.py: the public name lives here too."""
from .eqlinear import fast_equi_linear, eqlinear_clear_plan_cache, eqlinear_set_plan_cache, eqlinear_debug_info  # noqa: F401
