"""fuse_b200: B200 (sm_100a) implementation of the fused Ulysses projection operators.

The product is the CUDA library `libfuse_b200.so` behind the C ABI of include/fuse_b200.h;
this package is the thin Python mirror of the reference's operator interface used by the
tests and the benchmark.  There is no CPU or PyTorch fallback."""
from . import api  # noqa: F401
from ._native import lib  # noqa: F401
