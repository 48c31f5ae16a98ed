"""Module path of the reference's Triton kernels (``flex_gemm.kernels.triton``).
Nothing here is Triton: the package exists so that scripts which reach for
``kernels.triton.spconv.config.allow_tf32`` (the reference's own
tests/submconv/inf_ablation.py:20 does) find the switch where they expect it."""
from . import spconv  # noqa: F401
