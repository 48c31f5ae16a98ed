"""flexgemm_b200: sm_100a backend for 3D submanifold sparse convolution behind
the ``flex_gemm.ops.spconv`` interface.

    from flexgemm_b200.ops.spconv import sparse_submanifold_conv3d, set_algorithm

The compute path is hand-written CUDA in ``lib/libflexgemm_b200.so`` reached
through a C ABI (``include/flexgemm_b200.h``); there is no CPU fallback.
"""
from . import kernels, ops  # noqa: F401

__version__ = "0.1.0"
