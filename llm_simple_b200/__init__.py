"""B200-native attention hot path of llm_simple behind the reference's operator API.

The product is ``libgpu_ops.so`` (hand-written sm_100a CUDA kernels behind the C
ABI of ``include/gpu_ops.h``).  This package only loads it and offers thin
ctypes wrappers (``llm_simple_b200.ops``) that take torch tensors for device
memory and streams.  There is no CPU or PyTorch fallback: a missing library is
an ImportError at first use.
"""
from . import layer, ops  # noqa: F401

__all__ = ["ops", "layer"]
