"""b200norm: LayerNorm / RMSNorm forward + backward for NVIDIA B200 as hand-written sm_100a
CUDA kernels behind TritonHub's module and autograd.Function interface."""
from .functional import (_layernorm_bwd, _layernorm_fwd, _rmsnorm_bwd, _rmsnorm_fwd, finalize_dwdb, layernorm,
                         rmsnorm)
from .activations import GeLU, LayerNormGeLU, RMSNormGeLU, gelu, layernorm_gelu, rmsnorm_gelu
from .hostio import HostPipeline
from .modules import LayerNorm, RMSNorm
from .softmax import LogSoftmax, Softmax, Softmin
from .ops import norm, normalize

__all__ = ['LayerNorm', 'RMSNorm', 'layernorm', 'rmsnorm', 'finalize_dwdb', 'HostPipeline', 'GeLU', 'gelu',
           'LayerNormGeLU', 'RMSNormGeLU', 'layernorm_gelu', 'rmsnorm_gelu', 'Softmax', 'LogSoftmax', 'Softmin', 'norm', 'normalize']
__version__ = '0.1.0'
