"""Numeric mode switch for fp32 inputs.

``allow_tf32 = True``  : fp32 features/weights are multiplied as TF32 on the
                         tensor cores (fp32 accumulate) -- the reference default
                         on CUDA (flex_gemm/kernels/triton/spconv/config.py:6).
``allow_tf32 = False`` : fp32-accurate products (split-TF32 on the tensor cores).
16-bit inputs are unaffected.
"""
allow_tf32 = True
