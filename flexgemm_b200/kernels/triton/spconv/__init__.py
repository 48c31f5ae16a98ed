"""``flex_gemm.kernels.triton.spconv`` of the reference, reduced to what callers
poke from outside: the ``config`` module with ``allow_tf32``."""
from . import config  # noqa: F401
