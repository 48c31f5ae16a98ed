"""GPU tests of the fused forward epilogue (activation + residual in the conv
kernel): against the CPU oracle, and against the unfused sequence on the GPU.

Bars: residual-only results equal the unfused sequence bit for bit (same
roundings, no transcendental); with SiLU max|x - ref| <= 1e-2 * max|ref| against
the fp64 oracle; gradients within the same bound."""
import pytest
import torch

from oracle import submconv_oracle as orc

pytestmark = pytest.mark.gpu

DEV = torch.device("cuda:0")


@pytest.fixture(autouse=True)
def _defaults():
    from flexgemm_b200.kernels import config
    from flexgemm_b200.ops import spconv
    from flexgemm_b200.kernels import cuda as K
    spconv.set_algorithm(spconv.Algorithm.MASKED_IMPLICIT_GEMM_SPLITK)
    config.allow_tf32 = True
    # the fused epilogue is never split over the offsets; the unfused launches it is compared with bit for bit would be at
    # these small sizes (fp32 slabs added, then one rounding), so splitting is switched off here
    prev = K.set_conv_splitk(1)
    yield
    K.set_conv_splitk(prev)
    config.allow_tf32 = True


def max_err(a, b):
    a, b = a.detach().double().cpu(), b.detach().double().cpu()
    return (a - b).abs().max().item(), b.abs().max().item()


def problem(res, ci, co, dtype, seed):
    coords, feats, weight, bias, shape = orc.make_problem(res, ci, co, dtype, seed=seed)
    g = torch.Generator().manual_seed(seed + 100)
    residual = torch.randn(coords.shape[0], co, generator=g).to(feats.dtype)
    return coords, feats, weight, bias, residual, shape


@pytest.mark.parametrize("dtype", ["float16", "bfloat16", "float32"])
@pytest.mark.parametrize("activation,use_res", [(None, True), ("silu", False), ("silu", True)])
def test_fused_forward_matches_oracle_and_unfused(dtype, activation, use_res):
    from flexgemm_b200.ops import spconv
    coords, feats, weight, bias, residual, shape = problem(32, 64, 96, dtype, seed=3)
    f, w, b, r = feats.to(DEV), weight.to(DEV), bias.to(DEV), residual.to(DEV)
    c = coords.to(DEV)
    out, cache = spconv.sparse_submanifold_conv3d_fused(f, c, torch.Size(shape), w, b, activation=activation,
                                                        residual=r if use_res else None)
    # oracle in fp64 (no roundings): the tolerance covers the 16-bit roundings
    nbr = orc.neighbor_map(coords.numpy(), shape)
    ref = orc.residual_block_epilogue(orc.conv_forward(feats.double(), nbr, weight.double(), bias.double()), activation,
                                      residual.double() if use_res else None)
    err, scale = max_err(out, ref)
    bound = (1e-2 if dtype != "float32" else 2e-3) * scale  # fp32 features run on TF32 operands here
    assert err <= bound, (err, bound)
    # unfused sequence on the GPU
    y, _ = spconv.sparse_submanifold_conv3d(f, c, torch.Size(shape), w, b, neighbor_cache=cache)
    if activation == "silu":
        y = torch.nn.functional.silu(y)
    if use_res:
        y = y + r
    if activation is None:
        assert torch.equal(out, y)
    else:
        err, scale = max_err(out, y)
        assert err <= 4e-3 * scale, (err, scale)  # fast exp in the kernel against torch's expf, then one 16-bit rounding


def test_fused_forward_fp32_accurate_mode():
    from flexgemm_b200.kernels import config
    from flexgemm_b200.ops import spconv
    config.allow_tf32 = False
    coords, feats, weight, bias, residual, shape = problem(16, 32, 32, "float32", seed=5)
    out, _ = spconv.sparse_submanifold_conv3d_fused(feats.to(DEV), coords.to(DEV), torch.Size(shape), weight.to(DEV), bias.to(DEV),
                                                    activation="silu", residual=residual.to(DEV))
    nbr = orc.neighbor_map(coords.numpy(), shape)
    ref = orc.residual_block_epilogue(orc.conv_forward(feats.double(), nbr, weight.double(), bias.double()), "silu", residual.double())
    err, scale = max_err(out, ref)
    assert err <= 1e-4 * scale, (err, scale)


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
def test_fused_backward_matches_oracle(dtype):
    from flexgemm_b200.ops import spconv
    coords, feats, weight, bias, residual, shape = problem(32, 64, 64, dtype, seed=7)
    f = feats.to(DEV).requires_grad_(True)
    w = weight.to(DEV).requires_grad_(True)
    b = bias.to(DEV).requires_grad_(True)
    r = residual.to(DEV).requires_grad_(True)
    out, _ = spconv.sparse_submanifold_conv3d_fused(f, coords.to(DEV), torch.Size(shape), w, b, activation="silu", residual=r)
    g = torch.Generator().manual_seed(11)
    gout = torch.randn(out.shape, generator=g).to(out.dtype)
    out.backward(gout.to(DEV))

    nbr = orc.neighbor_map(coords.numpy(), shape)
    pre = orc.conv_forward(feats.double(), nbr, weight.double(), bias.double())
    gpre = orc.silu_backward(pre, gout.double())
    gin, gw, gb = orc.conv_backward(gpre, feats.double(), nbr, weight.double())
    for name, got, want in (("grad_feats", f.grad, gin), ("grad_weight", w.grad, gw), ("grad_bias", b.grad, gb),
                            ("grad_residual", r.grad, gout.double())):
        err, scale = max_err(got, want)
        assert err <= 1e-2 * scale, (name, err, scale)


def test_residual_only_gradient_and_no_conv_grads():
    from flexgemm_b200.ops import spconv
    coords, feats, weight, bias, residual, shape = problem(16, 32, 32, "float16", seed=9)
    r = residual.to(DEV).requires_grad_(True)
    out, cache = spconv.sparse_submanifold_conv3d_fused(feats.to(DEV), coords.to(DEV), torch.Size(shape), weight.to(DEV), None,
                                                        residual=r)
    out.sum().backward()
    assert torch.equal(r.grad, torch.ones_like(r))


def test_fused_rejects_bad_arguments():
    from flexgemm_b200.ops import spconv
    coords, feats, weight, bias, residual, shape = problem(8, 16, 16, "float16", seed=1)
    with pytest.raises(ValueError):
        spconv.sparse_submanifold_conv3d_fused(feats.to(DEV), coords.to(DEV), torch.Size(shape), weight.to(DEV), activation="gelu")
    with pytest.raises(AssertionError):
        spconv.sparse_submanifold_conv3d_fused(feats.to(DEV), coords.to(DEV), torch.Size(shape), weight.to(DEV),
                                               residual=residual.to(DEV)[:, :8].contiguous())
    with pytest.raises(NotImplementedError):
        spconv.sparse_submanifold_conv3d_fused(feats, coords, torch.Size(shape), weight)


def test_fused_empty_input():
    from flexgemm_b200.ops import spconv
    c = torch.zeros((0, 4), dtype=torch.int32, device=DEV)
    f = torch.zeros((0, 16), dtype=torch.float16, device=DEV)
    w = torch.zeros((16, 3, 3, 3, 16), dtype=torch.float16, device=DEV)
    out, _ = spconv.sparse_submanifold_conv3d_fused(f, c, torch.Size((1, 16, 8, 8, 8)), w, activation="silu", residual=f.clone())
    assert out.shape == (0, 16)
