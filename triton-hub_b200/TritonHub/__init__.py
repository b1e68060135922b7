"""Import-path shim: ``from TritonHub.Normalization import LayerNorm, RMSNorm`` and
``from TritonHub.Activations import GeLU`` / ``from TritonHub.Ops import norm, normalize`` resolve to the B200 kernels.  Nothing else of TritonHub exists here."""
from . import Activations, Normalization, Ops

__all__ = ['Normalization', 'Activations', 'Ops']
