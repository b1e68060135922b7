"""The part of TritonHub/Activations/__init__.py built on the B200 kernels: GeLU (the step after the
norm) and the row-wise Softmax family."""
from b200norm.activations import GeLU
from b200norm.softmax import LogSoftmax, Softmax, Softmin

__all__ = ['GeLU', 'Softmax', 'Softmin', 'LogSoftmax']
