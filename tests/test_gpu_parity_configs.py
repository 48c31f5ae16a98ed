"""GPU parity at the benchmarked configurations: the CUDA path against the CPU
oracle (never against itself) on the shapes the bench reports numbers for.

* headline: RES=256 shell, Ci=Co=256, fp16, random grad_out -- out and
  grad_feats on 4 096 random rows, ALL 27 offsets of grad_weight and grad_bias;
* the ends of the channel / dtype sweep: C=1024 fp16 and C=512 fp32 (TF32);
* the residual stack's shape: bf16, C=512, four RES=64 shells, two blocks;
* misaligned channel counts (Ci=3, Co=20) and the device status word.

The oracle's explicit algorithm needs N*27*C values per im2col, too much at the
headline size, so there it is evaluated where that is affordable: a row subset
for the row-wise outputs, and a chunked accumulation over the oracle's own
pair lists for the weight gradient.  fp16 products are exact in fp32, so chunks
are multiplied in fp32 and the chunk results are added in fp64.
Bars: 1e-2 * max|ref| for 16-bit types and TF32 (as stated for the path)."""
import numpy as np
import pytest
import torch

from oracle import submconv_oracle as orc

pytestmark = pytest.mark.gpu

DEV = torch.device("cuda:0")


@pytest.fixture(autouse=True)
def _masked_algorithm():
    from flexgemm_b200.kernels import config
    from flexgemm_b200.ops import spconv
    spconv.set_algorithm(spconv.Algorithm.MASKED_IMPLICIT_GEMM_SPLITK)
    spconv.set_hashmap_ratio(2.0)
    config.allow_tf32 = True
    yield
    config.allow_tf32 = True


def rel_err(got, want):
    return (got.detach().cpu().double() - want.double()).abs().max().item() / max(want.double().abs().max().item(), 1e-30)


def u32(t):
    return t.detach().cpu().view(torch.int32).numpy().view(np.uint32)


def gathered(x, idx, n):
    """[rows, V, C] fp64 with zeros where the neighbour is missing."""
    ok = (idx != 0xFFFFFFFF).unsqueeze(-1)
    return torch.where(ok, x.double()[idx.clamp(max=n - 1)], torch.zeros((), dtype=torch.float64))


def oracle_grad_weight(gout, feats, vs_i, vs_o, seg, chunk=16384):
    """[Co, V, Ci] fp64 from the oracle's pair lists: per offset, chunks of pairs
    multiplied in fp32 (exact products for 16-bit inputs), chunk sums added in fp64."""
    V = seg.shape[0] - 1
    Co, Ci = gout.shape[1], feats.shape[1]
    out = torch.zeros(Co, V, Ci, dtype=torch.float64)
    g32, x32 = gout.float(), feats.float()
    for v in range(V):
        acc = torch.zeros(Co, Ci, dtype=torch.float64)
        for s in range(int(seg[v]), int(seg[v + 1]), chunk):
            e = min(s + chunk, int(seg[v + 1]))
            o = torch.from_numpy(vs_o[s:e].astype(np.int64))
            i = torch.from_numpy(vs_i[s:e].astype(np.int64))
            acc += (g32[o].t() @ x32[i]).double()
        out[:, v, :] = acc
    return out


def test_headline_config_fwd_bwd_vs_oracle():
    """RES=256, Ci=Co=256, fp16 -- the configuration the headline number is quoted on."""
    from flexgemm_b200.kernels import cuda as K
    from flexgemm_b200.ops import spconv
    res, C = 256, 256
    coords_np = orc.shell_coords(res)
    n = coords_np.shape[0]
    shape = torch.Size((1, C, res, res, res))
    g = torch.Generator().manual_seed(2)
    feats = torch.randn(n, C, generator=g).half()
    weight = (torch.randn(C, 3, 3, 3, C, generator=g) / (27 * C) ** 0.5).half()
    bias = torch.randn(C, generator=g).half()
    gout = torch.randn(n, C, generator=g).half()

    f = feats.to(DEV).requires_grad_(True)
    w = weight.to(DEV).requires_grad_(True)
    b = bias.to(DEV).requires_grad_(True)
    out, cache = spconv.sparse_submanifold_conv3d(f, torch.from_numpy(coords_np).to(DEV), shape, w, b)
    out.backward(gout.to(DEV))
    torch.cuda.synchronize()
    K.check_status(DEV)

    ref = orc.neighbor_cache(coords_np, shape)
    nbr = ref["neighbor_map"]
    assert np.array_equal(u32(cache["neighbor_map"]), nbr)
    assert np.array_equal(u32(cache["valid_signal_i"]), ref["valid_signal_i"])
    assert np.array_equal(u32(cache["valid_signal_o"]), ref["valid_signal_o"])
    assert np.array_equal(u32(cache["valid_signal_seg"]), ref["valid_signal_seg"])
    assert int(ref["valid_signal_seg"][-1]) == 1712528

    # row-wise outputs on a random subset of rows, plus the first and last rows of the sorted order (tile edges)
    rng = np.random.default_rng(0)
    sidx = cache["sorted_idx"].cpu().numpy()
    rows_np = np.unique(np.concatenate([rng.choice(n, 4096, replace=False), sidx[:64], sidx[-64:]]))
    rows = torch.from_numpy(rows_np)
    sub = torch.from_numpy(nbr[rows_np].astype(np.int64))
    w64 = weight.double().reshape(C, 27, C)
    ref_out = torch.einsum("rvc,ovc->ro", gathered(feats, sub, n), w64) + bias.double()
    ref_gin = torch.einsum("rvo,ovc->rc", gathered(gout, torch.flip(sub, [1]), n), w64)
    assert rel_err(out[rows.to(DEV)], ref_out) <= 1e-2
    assert rel_err(f.grad[rows.to(DEV)], ref_gin) <= 1e-2

    # every offset of the weight gradient, and the bias gradient
    ref_gw = oracle_grad_weight(gout, feats, ref["valid_signal_i"], ref["valid_signal_o"], ref["valid_signal_seg"])
    got_gw = w.grad.reshape(C, 27, C)
    for v in range(27):
        assert rel_err(got_gw[:, v, :], ref_gw[:, v, :]) <= 1e-2, v
    assert rel_err(b.grad, gout.double().sum(0)) <= 1e-2


@pytest.mark.parametrize("res,c,dtype", [(32, 1024, "float16"), (32, 512, "float32"), (32, 1024, "bfloat16")])
def test_channel_sweep_ends_vs_oracle(res, c, dtype):
    """The widest points of the channel / dtype sweep: several output-channel tiles per
    row block in fprop / dgrad, several (output group, input tile) pairs per unit in wgrad."""
    from flexgemm_b200.kernels import cuda as K
    from flexgemm_b200.ops import spconv
    coords, feats, weight, bias, shape = orc.make_problem(res, c, c, dtype, seed=res + c)
    n = coords.shape[0]
    g = torch.Generator().manual_seed(5)
    gout = torch.randn(n, c, generator=g).to(feats.dtype)
    f = feats.to(DEV).requires_grad_(True)
    w = weight.to(DEV).requires_grad_(True)
    b = bias.to(DEV).requires_grad_(True)
    out, _ = spconv.sparse_submanifold_conv3d(f, coords.to(DEV), torch.Size(shape), w, b)
    out.backward(gout.to(DEV))
    torch.cuda.synchronize()
    K.check_status(DEV)
    nbr = orc.neighbor_map(coords.numpy(), shape)
    ref_out = orc.conv_forward(feats.double(), nbr, weight.double(), bias.double())
    ref_gin, ref_gw, ref_gb = orc.conv_backward(gout.double(), feats.double(), nbr, weight.double())
    for name, got, want in (("out", out, ref_out), ("grad_feats", f.grad, ref_gin), ("grad_weight", w.grad, ref_gw),
                            ("grad_bias", b.grad, ref_gb)):
        assert got.dtype == feats.dtype
        assert rel_err(got, want) <= 1e-2, (name, rel_err(got, want))


def test_residual_stack_shape_bf16_c512():
    """Four RES=64 shells, C=512, bf16, two residual blocks [conv, SiLU, conv] + skip
    with one shared neighbour cache -- the residual-stack workload's shape -- against
    the same network in fp32 torch ops on the CPU over the oracle's neighbour map."""
    from flexgemm_b200.kernels import cuda as K
    from flexgemm_b200.ops import spconv
    C, res, batch, blocks = 512, 64, 4, 2
    coords_np = orc.shell_coords(res, batch=batch, scales=(1.0,) * batch)
    n = coords_np.shape[0]
    assert n == 4 * 9968
    shape = torch.Size((batch, C, res, res, res))
    g = torch.Generator().manual_seed(15)
    x0 = torch.randn(n, C, generator=g).bfloat16()
    ws = [(torch.randn(C, 3, 3, 3, C, generator=g) / (27 * C) ** 0.5).bfloat16() for _ in range(2 * blocks)]
    bs = [(torch.randn(C, generator=g) * 0.1).bfloat16() for _ in range(2 * blocks)]

    coords = torch.from_numpy(coords_np).to(DEV)
    wd = [w.to(DEV).requires_grad_(True) for w in ws]
    bd = [b.to(DEV).requires_grad_(True) for b in bs]
    xd = x0.to(DEV).requires_grad_(True)
    cache, h = None, xd
    for blk in range(blocks):
        y, cache = spconv.sparse_submanifold_conv3d(h, coords, shape, wd[2 * blk], bd[2 * blk], cache)
        y = torch.nn.functional.silu(y)
        y, cache = spconv.sparse_submanifold_conv3d(y, coords, shape, wd[2 * blk + 1], bd[2 * blk + 1], cache)
        h = h + y
    h.float().mean().backward()
    torch.cuda.synchronize()
    K.check_status(DEV)

    nbr = torch.from_numpy(orc.neighbor_map(coords_np, shape).astype(np.int64))
    ok = nbr != 0xFFFFFFFF
    idx = nbr.clamp(max=n - 1)

    class Conv(torch.autograd.Function):
        """out = sum_v x[nbr[:, v]] W_v^T + b, one offset at a time (no im2col kept for the backward)."""

        @staticmethod
        def forward(ctx, x, w, b):
            ctx.save_for_backward(x, w)
            out = b.expand(n, -1).clone()
            for v in range(27):
                m = ok[:, v]
                out[m] += x[idx[m, v]] @ w[:, v, :].t()
            return out

        @staticmethod
        def backward(ctx, go):
            x, w = ctx.saved_tensors
            gx = torch.zeros_like(x)
            gw = torch.zeros_like(w)
            for v in range(27):
                m = ok[:, v]
                src = idx[m, v]
                gx.index_add_(0, src, go[m] @ w[:, v, :])
                gw[:, v, :] = go[m].t() @ x[src]
            return gx, gw, go.sum(0)

    wr = [w.float().reshape(C, 27, C).requires_grad_(True) for w in ws]
    br = [b.float().requires_grad_(True) for b in bs]
    xr = x0.float().requires_grad_(True)
    hr = xr
    for blk in range(blocks):
        y = torch.nn.functional.silu(Conv.apply(hr, wr[2 * blk], br[2 * blk]))
        hr = hr + Conv.apply(y, wr[2 * blk + 1], br[2 * blk + 1])
    hr.mean().backward()
    assert rel_err(h, hr) <= 2e-2          # four bf16 layers deep
    assert rel_err(xd.grad, xr.grad) <= 2e-2
    for a, r in zip(wd, wr):
        assert rel_err(a.grad.reshape(C, 27, C), r.grad) <= 2e-2
    for a, r in zip(bd, br):
        assert rel_err(a.grad, r.grad) <= 2e-2


@pytest.mark.parametrize("ci,co,dtype", [(3, 20, "float16"), (6, 32, "bfloat16"), (1, 5, "float32")])
def test_misaligned_channel_counts(ci, co, dtype):
    """First-layer channel counts (rows that are not whole 16-byte pieces) go through
    zero padding in the host wrappers; results have the caller's shapes."""
    from flexgemm_b200.kernels import cuda as K
    from flexgemm_b200.ops import spconv
    coords, feats, weight, bias, shape = orc.make_problem(16, ci, co, dtype, seed=40 + ci)
    g = torch.Generator().manual_seed(6)
    gout = torch.randn(coords.shape[0], co, generator=g).to(feats.dtype)
    f = feats.to(DEV).requires_grad_(True)
    w = weight.to(DEV).requires_grad_(True)
    b = bias.to(DEV).requires_grad_(True)
    out, _ = spconv.sparse_submanifold_conv3d(f, coords.to(DEV), torch.Size(shape), w, b)
    out.backward(gout.to(DEV))
    torch.cuda.synchronize()
    K.check_status(DEV)
    nbr = orc.neighbor_map(coords.numpy(), shape)
    ref_out = orc.conv_forward(feats.double(), nbr, weight.double(), bias.double())
    ref_gin, ref_gw, ref_gb = orc.conv_backward(gout.double(), feats.double(), nbr, weight.double())
    assert out.shape == (coords.shape[0], co) and f.grad.shape == feats.shape and w.grad.shape == weight.shape
    for name, got, want in (("out", out, ref_out), ("grad_feats", f.grad, ref_gin), ("grad_weight", w.grad, ref_gw),
                            ("grad_bias", b.grad, ref_gb)):
        assert rel_err(got, want) <= 1e-2, (name, rel_err(got, want))


def test_soft_error_reaches_the_caller_and_is_cleared():
    """A non-zero device status word makes every conv kernel return at once.  The
    word is set from the host here (no kernel fault involved): the conv calls must
    raise once the device has reported it, and work again afterwards."""
    from flexgemm_b200.kernels import cuda as K
    from flexgemm_b200.ops import spconv
    coords, feats, weight, bias, shape = orc.make_problem(16, 64, 64, "float16", seed=31)
    args = (feats.to(DEV), coords.to(DEV), torch.Size(shape), weight.to(DEV), bias.to(DEV))
    with torch.no_grad():
        good, cache = spconv.sparse_submanifold_conv3d(*args)
        torch.cuda.synchronize()
        K.check_status(DEV)
        K.status_word(DEV).fill_(2)          # what a kernel whose bounded wait ran out would leave
        torch.cuda.synchronize()
        with pytest.raises(RuntimeError, match="bounded barrier wait"):
            for _ in range(3):               # first call queues the look, a later one sees it
                spconv.sparse_submanifold_conv3d(*args, neighbor_cache=cache)
                torch.cuda.synchronize()
        torch.cuda.synchronize()
        assert int(K.status_word(DEV).item()) == 0
        again, _ = spconv.sparse_submanifold_conv3d(*args, neighbor_cache=cache)
        torch.cuda.synchronize()
        K.check_status(DEV)
        assert torch.equal(again, good)


@pytest.mark.parametrize("res,c,bands", [(32, 64, 64), (64, 128, 16), (48, 256, 5), (32, 64, 1)])
def test_wgrad_row_bands_vs_oracle(res, c, bands):
    """The weight gradient with the pair lists walked in a forced number of row
    bands (small inputs would otherwise get a single band): same result as the
    oracle, and -- being a different order of fp32 additions only -- within
    rounding of the single-band result."""
    from flexgemm_b200.kernels import cuda as K
    from flexgemm_b200.ops.spconv import SubMConv3dFunction as F
    coords, feats, weight, _, shape = orc.make_problem(res, c, c, "float16", seed=res + bands)
    g = torch.Generator().manual_seed(9)
    gout = torch.randn(coords.shape[0], c, generator=g).half()
    cache = F._compute_neighbor_cache(coords.to(DEV), torch.Size(shape), (3, 3, 3), (1, 1, 1), True)
    args = (gout.to(DEV), feats.to(DEV), cache["valid_signal_i"], cache["valid_signal_o"], cache["valid_signal_seg"])
    prev = K.set_wgrad_row_bands(bands)
    try:
        gw, gw32 = K.conv_wgrad(*args, want_f32=True, block_offsets=cache["pair_block_offsets"])
    finally:
        K.set_wgrad_row_bands(prev)
    plain, plain32 = K.conv_wgrad(*args, want_f32=True)          # no block offsets: one band
    torch.cuda.synchronize()
    K.check_status(DEV)
    nbr = orc.neighbor_map(coords.numpy(), shape)
    _, ref_gw, _ = orc.conv_backward(gout.double(), feats.double(), nbr, weight.double(), has_bias=False)
    ref = ref_gw.reshape(c, 27, c)
    assert rel_err(gw, ref) <= 1e-2 and rel_err(gw32, ref) <= 1e-2
    assert rel_err(gw32, plain32.double().cpu()) <= 1e-5


@pytest.mark.parametrize("res,batch,c,dtype", [(8, 1, 1024, "float16"), (16, 1, 256, "bfloat16"), (8, 2, 64, "float32"), (12, 1, 512, "float16")])
def test_splitk_of_small_launches_vs_oracle(res, batch, c, dtype):
    """Tiny inputs (a handful of row blocks): fprop and dgrad split every block's offsets
    into shares that run as separate work items.  Checked against the oracle with the
    automatic rule, with a forced odd share count and with splitting off, and the three
    must agree with each other to rounding."""
    from flexgemm_b200.kernels import cuda as K
    from flexgemm_b200.ops import spconv
    scales = (1.0,) * batch
    coords, feats, weight, bias, shape = orc.make_problem(res, c, c, dtype, seed=res + c, batch=batch, scales=scales)
    g = torch.Generator().manual_seed(3)
    gout = torch.randn(coords.shape[0], c, generator=g).to(feats.dtype)
    nbr = orc.neighbor_map(coords.numpy(), shape)
    ref_out = orc.conv_forward(feats.double(), nbr, weight.double(), bias.double())
    ref_gin, _, _ = orc.conv_backward(gout.double(), feats.double(), nbr, weight.double())
    results = []
    for setting in (0, 5, 1):
        prev = K.set_conv_splitk(setting)
        try:
            f = feats.to(DEV).requires_grad_(True)
            out, _ = spconv.sparse_submanifold_conv3d(f, coords.to(DEV), torch.Size(shape), weight.to(DEV), bias.to(DEV))
            out.backward(gout.to(DEV))
            torch.cuda.synchronize()
            K.check_status(DEV)
        finally:
            K.set_conv_splitk(prev)
        assert rel_err(out, ref_out) <= 1e-2, (setting, rel_err(out, ref_out))
        assert rel_err(f.grad, ref_gin) <= 1e-2, (setting, rel_err(f.grad, ref_gin))
        results.append((out.detach().float().cpu(), f.grad.float().cpu()))
    for o, gi in results[:2]:
        assert rel_err(o, results[2][0]) <= 4e-3 and rel_err(gi, results[2][1]) <= 4e-3


def test_reference_first_forward_case_res8_c1024_batch256():
    """The first case of the reference's forward test (its own shell rule, RES=8, 256 samples, C=1024, fp16)."""
    from flexgemm_b200.kernels import cuda as K
    from flexgemm_b200.ops import spconv
    res, c, batch = 8, 1024, 256
    base = orc.reference_sphere_coords(res)
    coords_np = np.concatenate([np.concatenate([np.full((base.shape[0], 1), b, np.int32), base[:, 1:]], axis=1) for b in range(batch)])
    coords_np = np.ascontiguousarray(coords_np.astype(np.int32))
    n = coords_np.shape[0]
    shape = torch.Size((batch, c, res, res, res))
    g = torch.Generator().manual_seed(8)
    feats = torch.randn(n, c, generator=g).half()
    weight = (torch.randn(c, 3, 3, 3, c, generator=g) / (27 * c) ** 0.5).half()
    bias = torch.randn(c, generator=g).half()
    with torch.no_grad():
        out, cache = spconv.sparse_submanifold_conv3d(feats.to(DEV), torch.from_numpy(coords_np).to(DEV), shape, weight.to(DEV), bias.to(DEV))
    torch.cuda.synchronize()
    K.check_status(DEV)
    nbr = orc.neighbor_map(coords_np, shape)
    assert np.array_equal(u32(cache["neighbor_map"]), nbr)
    rows_np = np.random.default_rng(1).choice(n, 3000, replace=False)
    sub = torch.from_numpy(nbr[rows_np].astype(np.int64))
    ref = torch.einsum("rvc,ovc->ro", gathered(feats, sub, n), weight.double().reshape(c, 27, c)) + bias.double()
    assert rel_err(out[torch.from_numpy(rows_np).to(DEV)], ref) <= 1e-2


@pytest.mark.parametrize("dtype,C", [(torch.float16, 256), (torch.bfloat16, 192), (torch.float16, 64), (torch.float16, 1024)])
def test_dgrad_reads_the_weight_as_stored(dtype, C):
    """dgrad of 16-bit types multiplies by the weight as stored (an MN-major operand); forcing the re-laid-out copy must
    give the same bits, and both must match the oracle."""
    from flexgemm_b200.kernels import cuda as K
    from flexgemm_b200.ops.spconv import SubMConv3dFunction as F
    coords = torch.from_numpy(orc.shell_coords(40)).to(DEV)
    n = coords.shape[0]
    shape = torch.Size((1, C, 40, 40, 40))
    g = torch.Generator(device="cpu").manual_seed(9)
    gout = torch.randn(n, C, generator=g).to(dtype).to(DEV)
    w = (torch.randn(C, 27, C, generator=g) / (27 * C) ** 0.5).to(dtype).to(DEV)
    cache = F._compute_neighbor_cache(coords, shape, (3, 3, 3), (1, 1, 1), True)
    tile = K.conv_tile_rows()
    args = (gout, w, cache["neighbor_map"], cache["sorted_idx"], cache.tile_masks(tile), cache.block_order(tile))
    prev = K.set_conv_dgrad_relayout(False)
    try:
        direct = K.conv_dgrad(*args)
        K.set_conv_dgrad_relayout(True)
        relaid = K.conv_dgrad(*args)
    finally:
        K.set_conv_dgrad_relayout(prev)
    K.check_status(DEV)
    assert torch.equal(direct.view(torch.int16), relaid.view(torch.int16))
    nbr = cache["neighbor_map"].cpu().view(torch.int32).numpy().view(np.uint32)
    rows = np.random.default_rng(3).choice(n, size=300, replace=False)
    wf = w.float().cpu().numpy().astype(np.float64)
    gf = gout.float().cpu().numpy().astype(np.float64)
    ref = np.zeros((rows.size, C))
    for k, r in enumerate(rows):
        for v in range(27):
            j = nbr[r, 26 - v]          # the row whose offset v is r
            if j != 0xFFFFFFFF:
                ref[k] += gf[j] @ wf[:, v, :]
    got = direct.float().cpu().numpy()[rows]
    assert np.abs(got - ref).max() <= 2e-2 * max(np.abs(ref).max(), 1e-6)
