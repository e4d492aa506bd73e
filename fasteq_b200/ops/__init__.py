"""Operator front-end with the reference's function names (fasteq/ops/__init__.py)."""
from .uniform1d_jit import fast_uniform1d_jit  # noqa: F401
from .eqlinear import fast_equi_linear  # noqa: F401
from .stc_uniform1d_jit import fast_stc_uniform1d_jit  # noqa: F401
