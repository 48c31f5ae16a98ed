"""The bias-gradient entry point for callers that cannot allocate device memory.

Some hosts hand a plug-in a fixed arena and forbid any further cudaMalloc, and
some service loops cannot afford the device-wide stall an allocation causes.
``fgb_subm_conv_bias_grad_noalloc`` serves them: its scratch is a fixed buffer
inside the library image, so the caller passes inputs and outputs only.  Here it
is called straight through the C ABI and compared with the ordinary entry point
(which takes a caller-provided workspace), twice in a row with different shapes,
because the built-in buffer keeps the previous call's contents.

This file sorts last on purpose: a run that stops at the first failure has
already run every other test."""
import pytest
import torch

from flexgemm_b200 import _cabi

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def _reference_entry(g, code):
    lib = _cabi.lib()
    n, co = g.shape
    nbytes = _cabi.check_size(lib.fgb_bias_grad_workspace_bytes(co), "workspace bytes")
    ws = torch.empty(nbytes // 4, dtype=torch.float32, device=DEV)
    gb = torch.empty(co, dtype=g.dtype, device=DEV)
    gb32 = torch.empty(co, dtype=torch.float32, device=DEV)
    stream = torch.cuda.current_stream(DEV).cuda_stream
    _cabi.check(lib.fgb_subm_conv_bias_grad(g.data_ptr(), gb.data_ptr(), gb32.data_ptr(), n, co, code, ws.data_ptr(), nbytes, stream),
                "fgb_subm_conv_bias_grad")
    return gb, gb32


def _noalloc_entry(g, code):
    lib = _cabi.lib()
    n, co = g.shape
    gb = torch.empty(co, dtype=g.dtype, device=DEV)       # outputs belong to the caller
    gb32 = torch.empty(co, dtype=torch.float32, device=DEV)
    stream = torch.cuda.current_stream(DEV).cuda_stream
    _cabi.check(lib.fgb_subm_conv_bias_grad_noalloc(g.data_ptr(), gb.data_ptr(), gb32.data_ptr(), n, co, code, stream),
                "fgb_subm_conv_bias_grad_noalloc")
    return gb, gb32


@pytest.mark.parametrize("dtype,code", [(torch.float16, _cabi.F16), (torch.bfloat16, _cabi.BF16), (torch.float32, _cabi.F32_TF32)])
def test_noalloc_bias_grad_matches_workspace_entry_twice(dtype, code):
    gen = torch.Generator().manual_seed(17)
    # the second call is smaller in both dimensions, so stale partial sums of the
    # first call remain in the shared buffer beside the ones it overwrites
    for n, co in ((70001, 256), (300, 72)):
        g = torch.randn(n, co, generator=gen).to(dtype).to(DEV)
        want, want32 = _reference_entry(g, code)
        got, got32 = _noalloc_entry(g, code)
        torch.cuda.synchronize()
        exact = g.double().sum(0)
        bound = 1e-2 * exact.abs().max().item()          # the tolerance of the conv parity tests
        assert (got.double() - want.double()).abs().max().item() <= bound
        assert (got32.double() - want32.double()).abs().max().item() <= bound
        assert (got32.double().cpu() - exact.cpu()).abs().max().item() <= bound
        # same kernels, same summation order: in fact identical
        assert torch.equal(got, want) and torch.equal(got32, want32)


@pytest.mark.parametrize("dtype,code", [(torch.float16, _cabi.F16), (torch.float32, _cabi.F32_TF32)])
def test_noalloc_at_the_channel_limit_allocates_nothing(dtype, code):
    """Co = 2048 with at least 592 rows uses the whole built-in buffer (16-bit rows
    take the vector path of the partial-sum kernel, fp32 rows the one-thread-per-
    column path), and the call itself must leave the amount of free device memory
    unchanged: outputs are made first, then the driver's own figure is read on both
    sides of the call."""
    lib = _cabi.lib()
    co = lib.fgb_noalloc_max_channels()
    n = 1500
    g = torch.randn(n, co, generator=torch.Generator().manual_seed(23)).to(dtype).to(DEV)
    want, want32 = _reference_entry(g, code)
    _noalloc_entry(g, code)                               # first call on this device may resolve the buffer's address
    gb = torch.empty(co, dtype=dtype, device=DEV)
    gb32 = torch.empty(co, dtype=torch.float32, device=DEV)
    stream = torch.cuda.current_stream(DEV).cuda_stream
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info(DEV)
    rc = lib.fgb_subm_conv_bias_grad_noalloc(g.data_ptr(), gb.data_ptr(), gb32.data_ptr(), n, co, code, stream)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info(DEV)
    _cabi.check(rc, "fgb_subm_conv_bias_grad_noalloc")
    assert free_after == free_before
    assert torch.equal(gb, want) and torch.equal(gb32, want32)
    exact = g.double().sum(0)
    assert (gb32.double() - exact).abs().max().item() <= 1e-2 * exact.abs().max().item()


def test_noalloc_rejects_sizes_beyond_the_builtin_buffer():
    lib = _cabi.lib()
    limit = lib.fgb_noalloc_max_channels()
    assert limit == 2048
    g = torch.zeros(4, 8, dtype=torch.float16, device=DEV)
    out = torch.zeros(8, dtype=torch.float16, device=DEV)
    rc = lib.fgb_subm_conv_bias_grad_noalloc(g.data_ptr(), out.data_ptr(), 0, 4, limit + 8, _cabi.F16, 0)
    assert rc == -7
    assert "built-in scratch" in _cabi.error_string(rc)
    with pytest.raises(ValueError):
        _cabi.check(rc, "fgb_subm_conv_bias_grad_noalloc")
