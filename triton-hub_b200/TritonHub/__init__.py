"""Import-path shim: ``from TritonHub.Normalization import LayerNorm, RMSNorm`` and
``from TritonHub.Activations import GeLU`` resolve to the B200 kernels.  Nothing else of TritonHub exists here."""
from . import Activations, Normalization

__all__ = ['Normalization', 'Activations']
