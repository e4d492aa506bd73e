"""e3nn-style modules over the three operators (the adapter layer the reference gets from a patched
cuequivariance_torch, which is not part of its tree)."""
from .modules import ChannelwiseTensorProduct, SO3Linear, SymmetricContraction  # noqa: F401
from ..ops.spherical_harmonics import SphericalHarmonics  # noqa: F401
