"""Ops: one function per kernel family. CUDA tensors run the sm_100a kernels, CPU tensors the fp32 reference."""
from . import reference  # noqa: F401
