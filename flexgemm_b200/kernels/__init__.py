"""Kernel-level interface: ``cuda`` mirrors the functions of the reference's
``flex_gemm.kernels.cuda`` extension that lie on the submanifold-conv path;
``config.allow_tf32`` is the switch the reference keeps in
``flex_gemm.kernels.triton.spconv.config`` (flex_gemm/kernels/triton/spconv/config.py:6)."""
from . import config, cuda, triton  # noqa: F401
