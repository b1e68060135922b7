"""The part of TritonHub/Activations/__init__.py that sits next to the norm path: GeLU."""
from b200norm.activations import GeLU

__all__ = ['GeLU']
