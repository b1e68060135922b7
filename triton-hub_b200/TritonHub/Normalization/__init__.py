"""Same export surface as TritonHub/Normalization/__init__.py:1-4."""
from b200norm.modules import LayerNorm, RMSNorm

__all__ = ['LayerNorm', 'RMSNorm']
