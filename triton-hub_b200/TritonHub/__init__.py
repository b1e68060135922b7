"""Import-path shim: ``from TritonHub.Normalization import LayerNorm, RMSNorm`` resolves to the
B200 kernels.  Only the Normalization package exists here."""
from . import Normalization

__all__ = ['Normalization']
