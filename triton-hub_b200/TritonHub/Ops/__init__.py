"""The part of TritonHub/Ops/__init__.py built on the B200 kernels: the row-wise p-norm and normalize."""
from b200norm.ops import norm, normalize

__all__ = ['normalize', 'norm']
