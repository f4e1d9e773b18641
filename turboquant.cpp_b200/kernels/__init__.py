"""Python entry points of the hand-written sm_100a kernels (sources in ../csrc)."""
from ._call import KernelError
