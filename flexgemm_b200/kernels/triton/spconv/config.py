"""The reference keeps its fp32 numeric switch at
``flex_gemm.kernels.triton.spconv.config.allow_tf32``
(flex_gemm/kernels/triton/spconv/config.py:6).  Here the switch lives in
``flexgemm_b200.kernels.config``; this module forwards attribute reads and
writes to it, so ``config.allow_tf32 = False`` set through either path is the
same setting."""
import sys
import types

from ... import config as _config


class _Forward(types.ModuleType):
    def __getattr__(self, name):
        return getattr(_config, name)

    def __setattr__(self, name, value):
        setattr(_config, name, value)


_self = sys.modules[__name__]
_fwd = _Forward(__name__, __doc__)
_fwd.__dict__.update({k: v for k, v in _self.__dict__.items() if k.startswith("__")})
sys.modules[__name__] = _fwd
