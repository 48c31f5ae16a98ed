"""GPU parity tests: every call goes through the C ABI (via the thin tensor
wrappers) and is compared with the CPU oracle and the golden fixtures.

Bars: integer outputs bit-exact (``sorted_idx``: a permutation under which the
binary code is non-decreasing, because the reference's argsort is unstable);
16-bit features and gradients within max|x - ref| <= 1e-2 * max|ref|; fp32 with
TF32 within the same bound; fp32 with TF32 disabled within 1e-4 relative."""
import os

import numpy as np
import pytest
import torch

from oracle import submconv_oracle as orc

pytestmark = pytest.mark.gpu

GOLD = os.path.join(os.path.dirname(__file__), "golden")


@pytest.fixture(scope="module")
def K():
    from flexgemm_b200.kernels import cuda
    return cuda


@pytest.fixture(autouse=True)
def _masked_algorithm():
    from flexgemm_b200.kernels import config
    from flexgemm_b200.ops import spconv
    spconv.set_algorithm(spconv.Algorithm.MASKED_IMPLICIT_GEMM_SPLITK)
    spconv.set_hashmap_ratio(2.0)
    config.allow_tf32 = True
    yield
    config.allow_tf32 = True


DEV = torch.device("cuda:0")


def u32(t):
    return t.detach().cpu().view(torch.int32).numpy().view(np.uint32)


def build_cache(coords_np, shape, ksize=(3, 3, 3), dil=(1, 1, 1), needs_grad=True):
    from flexgemm_b200.ops.spconv import SubMConv3dFunction
    coords = torch.from_numpy(np.ascontiguousarray(coords_np)).to(DEV)
    return SubMConv3dFunction._compute_neighbor_cache(coords, torch.Size([int(s) for s in shape]), ksize, dil, needs_grad)


def check_cache(cache, ref, V, needs_grad=True, blocks=(128, 32)):
    nbr = u32(cache["neighbor_map"])
    assert np.array_equal(nbr, ref["neighbor_map"])
    assert np.array_equal(cache["gray_code"].cpu().numpy(), ref["gray_code"])
    sidx = cache["sorted_idx"].cpu().numpy()
    assert cache["sorted_idx"].dtype == torch.int64
    assert orc.is_valid_sorted_idx(sidx, ref["binary_code"])
    if needs_grad:
        assert np.array_equal(u32(cache["valid_signal_seg"]), ref["valid_signal_seg"])
        assert np.array_equal(u32(cache["valid_signal_i"]), ref["valid_signal_i"])
        assert np.array_equal(u32(cache["valid_signal_o"]), ref["valid_signal_o"])
    for b in blocks:
        vk, seg = orc.valid_kernel(ref["gray_code"], sidx, b)
        assert np.array_equal(u32(cache.tile_masks(b)), orc.tile_masks(ref["gray_code"], sidx, b))
        assert np.array_equal(cache.valid_kernel_callback(b).cpu().numpy(), vk)
        assert np.array_equal(cache.valid_kernel_seg_callback(b).cpu().numpy(), seg)


# ----------------------------------------------------------------------------
# neighbour map + post-processing: bit-exact
# ----------------------------------------------------------------------------
MAPS = np.load(os.path.join(GOLD, "neighbor_maps.npz"))


@pytest.mark.parametrize("name", sorted({k.split("/")[0] for k in MAPS.files}))
def test_neighbor_map_golden(name, K):
    coords = MAPS[name + "/coords"]
    shape = MAPS[name + "/shape"]
    ks, dil = tuple(int(x) for x in MAPS[name + "/ksize"]), tuple(int(x) for x in MAPS[name + "/dilation"])
    cache = build_cache(coords, shape, ks, dil)
    assert np.array_equal(u32(cache["neighbor_map"]), MAPS[name + "/neighbor_map"])
    check_cache(cache, orc.neighbor_cache(coords, shape, ks, dil), ks[0] * ks[1] * ks[2])


@pytest.mark.parametrize("res,batch", [(32, 1), (64, 2), (128, 1)])
def test_cache_vs_oracle_shells(res, batch, K):
    scales = tuple(1.0 - 0.15 * i for i in range(batch))
    coords = orc.shell_coords(res, batch=batch, scales=scales)
    shape = (batch, 0, res, res, res)
    for needs_grad in (True, False):
        cache = build_cache(coords, shape, needs_grad=needs_grad)
        assert ("valid_signal_i" in cache) == needs_grad
        check_cache(cache, orc.neighbor_cache(coords, shape), 27, needs_grad)


def test_cache_64bit_keys(K):
    """B*W*H*D >= 2^32 selects the 64-bit key table; voxels placed near the far
    corner of the last sample so that keys really exceed 32 bits."""
    rng = np.random.default_rng(5)
    base = orc.shell_coords(16)
    parts = []
    for b, off in ((0, 0), (7, 1024 - 16)):
        c = base.copy()
        c[:, 0] = b
        c[:, 1:] += off
        parts.append(c)
    coords = np.concatenate(parts)
    coords = np.ascontiguousarray(coords[rng.permutation(coords.shape[0])])
    shape = (8, 0, 1024, 1024, 1024)
    from flexgemm_b200.ops.utils import hashmap_key_bits
    assert hashmap_key_bits(shape) == 64
    check_cache(build_cache(coords, shape), orc.neighbor_cache(coords, shape), 27)


def test_cache_tight_table_and_unsorted(K):
    from flexgemm_b200.ops import spconv
    rng = np.random.default_rng(9)
    coords = orc.shell_coords(32)
    coords = np.ascontiguousarray(coords[rng.permutation(coords.shape[0])])
    spconv.set_hashmap_ratio(1.0)  # every slot used: probes wrap around
    check_cache(build_cache(coords, (1, 0, 32, 32, 32)), orc.neighbor_cache(coords, (1, 0, 32, 32, 32)), 27)


def test_sorted_and_hash_paths_agree(K):
    """Input in ascending key order takes the table-free path, anything else the
    hash table: the same voxels shuffled give the same map up to the row
    permutation, and sorted 64-bit keys work too."""
    rng = np.random.default_rng(11)
    base = orc.shell_coords(40, batch=2, scales=(1.0, 0.6))
    shape = (2, 0, 40, 40, 40)
    ref = orc.neighbor_cache(base, shape)
    check_cache(build_cache(base, shape), ref, 27)                       # sorted
    perm = rng.permutation(base.shape[0])
    shuffled = np.ascontiguousarray(base[perm])
    shuffled_cache = build_cache(shuffled, shape)                        # hash path
    check_cache(shuffled_cache, orc.neighbor_cache(shuffled, shape), 27)  # pair lists gathered from the map
    got = u32(shuffled_cache["neighbor_map"])
    inv = np.empty_like(perm)
    inv[perm] = np.arange(perm.size)
    want = ref["neighbor_map"][perm]                                     # rows follow the voxels ...
    want = np.where(want == orc.INVALID, orc.INVALID, inv[np.minimum(want, perm.size - 1)].astype(np.uint32))  # ... so do the entries
    assert np.array_equal(got, want)
    # sorted coordinates whose flat index needs 64 bits
    far = base.copy()
    far[:, 0] += 6
    far[:, 1:] += 1024 - 40
    big = (8, 0, 1024, 1024, 1024)
    check_cache(build_cache(far, big), orc.neighbor_cache(far, big), 27)


def test_pair_lists_with_and_without_the_map(K):
    """Rows in key order: the build leaves 0 in the word after the segment table and the pair lists then come from the
    masks alone; the same call without that word gathers them from the map.  Both must be the oracle's lists.  Shuffled
    rows leave a non-zero word."""
    from flexgemm_b200.ops import spconv, utils
    base = orc.shell_coords(48, batch=2, scales=(1.0, 0.7))
    shape = (2, 0, 48, 48, 48)
    for ksize, dil in (((3, 3, 3), (1, 1, 1)), ((3, 1, 5), (2, 1, 1))):
        V = ksize[0] * ksize[1] * ksize[2]
        ref = orc.neighbor_cache(base, shape, ksize, dil)
        coords = torch.from_numpy(base).to(DEV)
        n = coords.shape[0]
        slots = max(int(spconv.HASHMAP_RATIO * n), n, 1)
        table, key_bits = utils.init_table(torch.Size(shape), slots, coords.device)
        built = K.subm_build_neighbor_map(coords, torch.Size(shape), ksize, dil, table, key_bits, slots)
        assert int(built["order_flag"].cpu().view(torch.int32).item()) == 0
        pairs = int(ref["valid_signal_seg"][V])
        for flag in (built["order_flag"], None):
            vs_i, vs_o = K.valid_signal(built["neighbor_map"], built["gray_code"], built["block_offsets"], built["valid_signal_seg"],
                                        pairs, flag)
            assert np.array_equal(u32(vs_i), ref["valid_signal_i"]) and np.array_equal(u32(vs_o), ref["valid_signal_o"])
    rng = np.random.default_rng(5)
    shuffled = torch.from_numpy(np.ascontiguousarray(base[rng.permutation(base.shape[0])])).to(DEV)
    table, key_bits = utils.init_table(torch.Size(shape), slots, shuffled.device)
    built = K.subm_build_neighbor_map(shuffled, torch.Size(shape), (3, 3, 3), (1, 1, 1), table, key_bits, slots)
    assert int(built["order_flag"].cpu().view(torch.int32).item()) != 0


def test_sorted_path_runs_much_longer_than_a_block(K):
    """A sparse plane between two dense ones: the 256 voxels of a block span the
    whole sparse plane, so the run of rows of the next plane that can hold their
    neighbours is thousands of rows long (and most of those rows find nothing)."""
    g = np.arange(64)
    yy, zz = np.meshgrid(g, g, indexing="ij")
    dense = np.stack([yy.ravel(), zz.ravel()], axis=1)
    sparse = dense[(dense[:, 0] % 5 == 0) & (dense[:, 1] % 3 == 0)]
    planes = []
    for x, pts in ((10, dense), (11, sparse), (12, dense), (13, sparse[::7]), (14, dense)):
        planes.append(np.concatenate([np.zeros((len(pts), 1), int), np.full((len(pts), 1), x), pts], axis=1))
    coords = np.ascontiguousarray(np.concatenate(planes).astype(np.int32))
    shape = (1, 0, 64, 64, 64)
    assert np.all(np.diff(((coords[:, 1].astype(np.int64) * 64) + coords[:, 2]) * 64 + coords[:, 3]) > 0)
    check_cache(build_cache(coords, shape), orc.neighbor_cache(coords, shape), 27)


def test_cache_deterministic(K):
    coords = orc.shell_coords(64)
    a = build_cache(coords, (1, 0, 64, 64, 64))
    b = build_cache(coords, (1, 0, 64, 64, 64))
    for k in ("neighbor_map", "gray_code", "sorted_idx", "valid_signal_i", "valid_signal_o", "valid_signal_seg"):
        assert torch.equal(a[k], b[k]), k


def test_empty_and_tiny_inputs(K):
    cache = build_cache(np.zeros((0, 4), np.int32), (1, 0, 8, 8, 8))
    assert cache["neighbor_map"].shape == (0, 27)
    assert cache["valid_signal_i"].shape == (0,)
    assert np.array_equal(u32(cache["valid_signal_seg"]), np.zeros(28, np.uint32))
    one = np.array([[0, 3, 3, 3]], np.int32)
    check_cache(build_cache(one, (1, 0, 8, 8, 8)), orc.neighbor_cache(one, (1, 0, 8, 8, 8)), 27)


# ----------------------------------------------------------------------------
# features and gradients
# ----------------------------------------------------------------------------
def rel_err(got, want):
    return (got.detach().cpu().double() - want.double()).abs().max().item() / max(want.double().abs().max().item(), 1e-30)


def run_conv(coords, feats, weight, bias, shape, grad_out=None, cache=None):
    from flexgemm_b200.ops import spconv
    f = feats.to(DEV).requires_grad_(True)
    w = weight.to(DEV).requires_grad_(True)
    b = bias.to(DEV).requires_grad_(True) if bias is not None else None
    out, cache = spconv.sparse_submanifold_conv3d(f, coords.to(DEV), torch.Size(shape), w, b, cache)
    if grad_out is None:
        out.sum().backward()
    else:
        out.backward(grad_out.to(DEV))
    torch.cuda.synchronize()
    from flexgemm_b200.kernels import cuda
    cuda.check_status(DEV)
    return out, f.grad, w.grad, (b.grad if b is not None else None), cache


def oracle_conv(coords, feats, weight, bias, shape, grad_out=None):
    nbr = orc.neighbor_map(coords.numpy(), shape)
    f, w = feats.double(), weight.double()
    b = bias.double() if bias is not None else None
    out = orc.conv_forward(f, nbr, w, b)
    g = torch.ones_like(out) if grad_out is None else grad_out.double()
    gin, gw, gb = orc.conv_backward(g, f, nbr, w, has_bias=bias is not None)
    return out, gin, gw, gb


CONV_CASES = [
    # res, ci, co, dtype, batch, tolerance
    (16, 64, 64, "float16", 1, 1e-2),
    (32, 64, 64, "float16", 1, 1e-2),
    (32, 128, 256, "float16", 1, 1e-2),
    (32, 256, 128, "bfloat16", 1, 1e-2),
    (24, 32, 48, "float16", 2, 1e-2),
    (16, 72, 40, "float16", 1, 1e-2),     # channel counts that are not multiples of 64
    (32, 32, 32, "float32", 1, 1e-2),     # TF32
    (16, 320, 512, "float16", 1, 1e-2),   # more than one output-channel tile / accumulator group
    (64, 256, 256, "float16", 1, 1e-2),
]


@pytest.mark.parametrize("res,ci,co,dtype,batch,tol", CONV_CASES)
def test_conv_fwd_bwd_vs_oracle(res, ci, co, dtype, batch, tol, K):
    scales = tuple(1.0 - 0.2 * i for i in range(batch))
    coords, feats, weight, bias, shape = orc.make_problem(res, ci, co, dtype, seed=res + ci + co, batch=batch, scales=scales)
    g = torch.Generator().manual_seed(1)
    grad_out = torch.randn(coords.shape[0], co, generator=g).to(feats.dtype)
    got = run_conv(coords, feats, weight, bias, shape, grad_out)
    want = oracle_conv(coords, feats, weight, bias, shape, grad_out)
    for name, a, b in zip(("out", "grad_feats", "grad_weight", "grad_bias"), got[:4], want):
        assert a.dtype == feats.dtype and a.shape == b.shape, name
        assert rel_err(a, b) <= tol, (name, rel_err(a, b))


@pytest.mark.parametrize("res,ci,co,batch", [(32, 32, 32, 1), (16, 64, 48, 2), (24, 128, 256, 1)])
def test_conv_fp32_without_tf32(res, ci, co, batch, K):
    """allow_tf32 = False: fp32-accurate products (split-TF32), <= 1e-4 relative."""
    from flexgemm_b200.kernels import config
    config.allow_tf32 = False
    scales = tuple(1.0 - 0.2 * i for i in range(batch))
    coords, feats, weight, bias, shape = orc.make_problem(res, ci, co, "float32", seed=res + ci, batch=batch, scales=scales)
    g = torch.Generator().manual_seed(2)
    grad_out = torch.randn(coords.shape[0], co, generator=g)
    got = run_conv(coords, feats, weight, bias, shape, grad_out)
    want = oracle_conv(coords, feats, weight, bias, shape, grad_out)
    for name, a, b in zip(("out", "grad_feats", "grad_weight", "grad_bias"), got[:4], want):
        assert a.dtype == torch.float32
        assert rel_err(a, b) <= 1e-4, (name, rel_err(a, b))
    # and it is really tighter than the TF32 mode on the same inputs
    config.allow_tf32 = True
    tf32 = run_conv(coords, feats, weight, bias, shape, grad_out)
    assert rel_err(tf32[0], want[0]) > rel_err(got[0], want[0])


CONV = np.load(os.path.join(GOLD, "conv_explicit.npz"))


@pytest.mark.parametrize("name", ["r16_c32_c32_f32", "r12_c64_c32_f16", "r8_c16_c24_f32"])
def test_conv_vs_reference_golden(name, K):
    """Against outputs of the reference's own explicit path (fixture)."""
    t = {k: torch.from_numpy(CONV[f"{name}/{k}"]) for k in
         ("coords", "feats", "weight", "bias", "out", "grad_out", "grad_feats", "grad_weight", "grad_bias")}
    shape = CONV[name + "/shape"].tolist()
    got = run_conv(t["coords"], t["feats"], t["weight"], t["bias"], shape, t["grad_out"])
    for key, a in zip(("out", "grad_feats", "grad_weight", "grad_bias"), got[:4]):
        assert rel_err(a, t[key]) <= 1e-2, (key, rel_err(a, t[key]))


def test_conv_without_bias_and_cache_reuse(K):
    coords, feats, weight, _, shape = orc.make_problem(16, 64, 64, "float16", seed=21)
    out, gin, gw, gb, cache = run_conv(coords, feats, weight, None, shape)
    want = oracle_conv(coords, feats, weight, None, shape)
    assert gb is None
    assert rel_err(out, want[0]) <= 1e-2 and rel_err(gin, want[1]) <= 1e-2 and rel_err(gw, want[2]) <= 1e-2
    out2, gin2, gw2, _, cache2 = run_conv(coords, feats, weight, None, shape, cache=cache)
    assert cache2 is cache
    assert torch.equal(out, out2) and torch.equal(gin, gin2) and torch.equal(gw, gw2)  # deterministic


def test_no_grad_forward_builds_inference_cache(K):
    from flexgemm_b200.ops import spconv
    coords, feats, weight, bias, shape = orc.make_problem(16, 64, 64, "float16", seed=22)
    with torch.no_grad():
        out, cache = spconv.sparse_submanifold_conv3d(feats.to(DEV), coords.to(DEV), torch.Size(shape), weight.to(DEV), bias.to(DEV))
    assert "valid_signal_i" not in cache
    assert rel_err(out, oracle_conv(coords, feats, weight, bias, shape)[0]) <= 1e-2


def test_all_implicit_algorithms_agree(K):
    from flexgemm_b200.ops import spconv
    coords, feats, weight, bias, shape = orc.make_problem(16, 64, 64, "float16", seed=23)
    outs = []
    for alg in (spconv.Algorithm.IMPLICIT_GEMM, spconv.Algorithm.IMPLICIT_GEMM_SPLITK, spconv.Algorithm.MASKED_IMPLICIT_GEMM,
                spconv.Algorithm.MASKED_IMPLICIT_GEMM_SPLITK, spconv.Algorithm.EXPLICIT_GEMM):
        spconv.set_algorithm(alg)
        outs.append(run_conv(coords, feats, weight, bias, shape)[:4])
    want = oracle_conv(coords, feats, weight, bias, shape)
    for o in outs:
        for a, b in zip(o, want):
            assert rel_err(a, b) <= 1e-2
    for o in outs[1:4]:
        for a, b in zip(o, outs[0]):
            assert torch.equal(a, b)


def test_linearity_at_benchmark_size(K):
    """Size-independent property at the headline size (RES=256, C=256 fp16):
    conv(a + b) == conv(a) + conv(b) without bias, and the centre-only weight
    reproduces a plain matmul of the features."""
    from flexgemm_b200.ops import spconv
    coords = torch.from_numpy(orc.shell_coords(256)).to(DEV)
    n = coords.shape[0]
    shape = torch.Size((1, 256, 256, 256, 256))
    g = torch.Generator(device="cpu").manual_seed(3)
    a = torch.randn(n, 256, generator=g).half().to(DEV)
    b = torch.randn(n, 256, generator=g).half().to(DEV)
    w = (torch.randn(256, 3, 3, 3, 256, generator=g) / (27 * 256) ** 0.5).half().to(DEV)
    with torch.no_grad():
        ya, cache = spconv.sparse_submanifold_conv3d(a, coords, shape, w)
        yb, _ = spconv.sparse_submanifold_conv3d(b, coords, shape, w, None, cache)
        yab, _ = spconv.sparse_submanifold_conv3d((a.float() + b.float()).half(), coords, shape, w, None, cache)
        scale = yab.float().abs().max().item()
        assert (yab.float() - ya.float() - yb.float()).abs().max().item() <= 2e-2 * scale
        wc = torch.zeros_like(w)
        wc[:, 1, 1, 1, :] = w[:, 1, 1, 1, :]
        yc, _ = spconv.sparse_submanifold_conv3d(a, coords, shape, wc, None, cache)
        ref = a.float() @ w[:, 1, 1, 1, :].float().t()
        assert (yc.float() - ref).abs().max().item() <= 1e-2 * ref.abs().max().item()
    K.check_status(DEV)


def test_large_sample_res1024_c64(K):
    """One sample of the RES=1024 configuration (about 2.7 M voxels, C=64 fp16):
    neighbour map bit-exact against the oracle, and forward / feature gradient
    checked on a random subset of rows (the dense oracle would need 36 GB), the
    weight gradient through linearity of the whole pass."""
    from flexgemm_b200.ops import spconv
    res, C = 1024, 64
    coords_np = orc.shell_coords(res)
    n = coords_np.shape[0]
    assert n > 2_500_000
    shape = torch.Size((1, C, res, res, res))
    coords = torch.from_numpy(coords_np).to(DEV)
    g = torch.Generator().manual_seed(4)
    feats = torch.randn(n, C, generator=g).half()
    weight = (torch.randn(C, 3, 3, 3, C, generator=g) / (27 * C) ** 0.5).half()
    bias = torch.randn(C, generator=g).half()
    f = feats.to(DEV).requires_grad_(True)
    w = weight.to(DEV).requires_grad_(True)
    b = bias.to(DEV).requires_grad_(True)
    out, cache = spconv.sparse_submanifold_conv3d(f, coords, shape, w, b)
    gout = torch.randn(n, C, generator=g).half()
    out.backward(gout.to(DEV))
    torch.cuda.synchronize()
    K.check_status(DEV)
    nbr = orc.neighbor_map(coords_np, shape)
    assert np.array_equal(u32(cache["neighbor_map"]), nbr)
    assert int(u32(cache["valid_signal_seg"])[-1]) == orc.useful_pairs(nbr)
    rows = torch.from_numpy(np.random.default_rng(0).choice(n, 4000, replace=False))
    sub = torch.from_numpy(nbr[rows.numpy()].astype(np.int64))
    w64 = weight.double().reshape(C, 27, C)
    def gathered(x, idx):                       # [rows, 27, C] with zeros for missing neighbours
        ok = (idx != 0xFFFFFFFF).unsqueeze(-1)
        return torch.where(ok, x.double()[idx.clamp(max=n - 1)], torch.zeros((), dtype=torch.float64))
    ref_out = torch.einsum("rvc,ovc->ro", gathered(feats, sub), w64) + bias.double()
    ref_gin = torch.einsum("rvo,ovc->rc", gathered(gout, torch.flip(sub, [1])), w64)
    assert rel_err(out[rows.to(DEV)], ref_out) <= 1e-2
    assert rel_err(f.grad[rows.to(DEV)], ref_gin) <= 1e-2
    # weight gradient: centre offset is a plain X^T G product
    ref_gw_centre = gout.double().t() @ feats.double()
    assert rel_err(w.grad[:, 1, 1, 1, :], ref_gw_centre) <= 1e-2
    assert rel_err(b.grad, gout.double().sum(0)) <= 1e-2


def test_residual_stack_with_shared_cache(K):
    """Two residual blocks [conv, SiLU, conv] + skip over a batch of shells, bf16,
    the neighbour cache built once and passed to every layer (the way a network
    uses the op); loss = mean of the output.  Checked against the same network
    written with plain torch ops in fp64 on the CPU (gather through the oracle's
    neighbour map, autograd for the gradients)."""
    from flexgemm_b200.ops import spconv
    C, res, batch = 64, 16, 2
    coords_np = orc.shell_coords(res, batch=batch, scales=(1.0, 0.8))
    n = coords_np.shape[0]
    shape = torch.Size((batch, C, res, res, res))
    g = torch.Generator().manual_seed(8)
    x0 = torch.randn(n, C, generator=g).bfloat16()
    ws = [(torch.randn(C, 3, 3, 3, C, generator=g) / (27 * C) ** 0.5).bfloat16() for _ in range(4)]
    bs = [torch.randn(C, generator=g).bfloat16() * 0.1 for _ in range(4)]

    # device
    coords = torch.from_numpy(coords_np).to(DEV)
    wd = [w.to(DEV).requires_grad_(True) for w in ws]
    bd = [b.to(DEV).requires_grad_(True) for b in bs]
    xd = x0.to(DEV).requires_grad_(True)
    cache, h = None, xd
    for blk in range(2):
        y, cache = spconv.sparse_submanifold_conv3d(h, coords, shape, wd[2 * blk], bd[2 * blk], cache)
        y = torch.nn.functional.silu(y)
        y, cache = spconv.sparse_submanifold_conv3d(y, coords, shape, wd[2 * blk + 1], bd[2 * blk + 1], cache)
        h = h + y
    h.float().mean().backward()
    torch.cuda.synchronize()
    K.check_status(DEV)

    # reference
    nbr = torch.from_numpy(orc.neighbor_map(coords_np, shape).astype(np.int64))
    ok = (nbr != 0xFFFFFFFF).unsqueeze(-1)
    idx = nbr.clamp(max=n - 1)
    def conv(x, w, b):
        col = torch.where(ok, x[idx], torch.zeros((), dtype=x.dtype)).reshape(n, -1)
        return col @ w.reshape(C, -1).t() + b
    wr = [w.double().requires_grad_(True) for w in ws]
    br = [b.double().requires_grad_(True) for b in bs]
    xr = x0.double().requires_grad_(True)
    hr = xr
    for blk in range(2):
        y = torch.nn.functional.silu(conv(hr, wr[2 * blk], br[2 * blk]))
        hr = hr + conv(y, wr[2 * blk + 1], br[2 * blk + 1])
    hr.mean().backward()
    assert rel_err(h, hr) <= 2e-2          # four bf16 layers deep
    assert rel_err(xd.grad, xr.grad) <= 2e-2
    for a, b in zip(wd + bd, wr + br):
        assert rel_err(a.grad, b.grad) <= 2e-2


def test_sharded_backward_on_the_kernels_matches_the_sum_over_shards(K):
    """The multi-GPU backward (fp32 parameter gradients, one all-reduce, cast) run
    as a single rank per shard on one GPU: summing the shards' fp32 gradients by
    hand must give the unsharded gradient, and each shard's feature gradient must
    equal the rows of the unsharded one."""
    from flexgemm_b200 import sharding
    from flexgemm_b200.ops.spconv import SubMConv3dFunction as F
    coords_np, feats, weight, bias, shape = orc.make_problem(24, 64, 64, "float16", seed=12, batch=3, scales=(1.0, 0.8, 0.6))
    g = torch.Generator().manual_seed(2)
    gout = torch.randn(coords_np.shape[0], 64, generator=g).half()
    nbr = orc.neighbor_map(coords_np.numpy(), shape)
    ref_gin, ref_gw, ref_gb = orc.conv_backward(gout.double(), feats.double(), nbr, weight.double())
    w, b = weight.to(DEV), bias.to(DEV)
    total_w = torch.zeros_like(ref_gw)
    total_b = torch.zeros_like(ref_gb)
    for rank in range(2):
        c, f, lshape, rows = sharding.local_shard(coords_np, feats, shape, rank, 2)
        cache = F._compute_neighbor_cache(c.to(DEV), lshape, (3, 3, 3), (1, 1, 1), True)
        gin, gw, gb = sharding.sharded_backward(gout[rows].to(DEV), f.to(DEV), cache, w, b)   # no process group: world of one
        assert gw.dtype == torch.float16 and gw.shape == weight.shape
        assert rel_err(gin, ref_gin[rows]) <= 1e-2
        total_w += gw.double().cpu()
        total_b += gb.double().cpu()
    assert rel_err(total_w, ref_gw) <= 1e-2 and rel_err(total_b, ref_gb) <= 1e-2


@pytest.mark.parametrize("ksize,dil", [((3, 3, 3), (1, 1, 1)), ((3, 3, 3), (2, 1, 3)), ((1, 1, 5), (1, 1, 1)), ((5, 1, 5), (1, 1, 2)),
                                       ((3, 1, 3), (1, 2, 9))])
def test_sorted_input_with_long_columns(ksize, dil, K):
    """Rows in key order whose (b, x, y) columns are long (a dense slab: up to 48 voxels per
    column, searched by bisection) next to short and empty ones, for stencils of several
    extents and dilations -- the table-free path serves every odd stencil."""
    rng = np.random.default_rng(21)
    W, H, D = 12, 10, 48
    dense = np.stack(np.meshgrid(np.arange(3, 9), np.arange(2, 8), np.arange(D), indexing="ij"), -1).reshape(-1, 3)
    sparse = np.stack(np.meshgrid(np.arange(W), np.arange(H), np.arange(D), indexing="ij"), -1).reshape(-1, 3)
    sparse = sparse[rng.random(sparse.shape[0]) < 0.07]
    pts = np.unique(np.concatenate([dense, sparse]), axis=0)            # lexicographic (x, y, z)
    coords = np.concatenate([np.concatenate([np.full((pts.shape[0], 1), b), pts], axis=1) for b in range(2)]).astype(np.int32)
    shape = (2, 0, W, H, D)
    check_cache(build_cache(coords, shape, ksize, dil), orc.neighbor_cache(coords, shape, ksize, dil), ksize[0] * ksize[1] * ksize[2])


POST = np.load(os.path.join(GOLD, "postprocess.npz"))


@pytest.mark.parametrize("name", sorted({k.split("/")[0] for k in POST.files}))
def test_cache_vs_reference_cuda_output(name, K):
    """The whole neighbour cache against what the reference's own compiled CUDA functions produced
    for the same coordinates (fixture: tests/golden/make_golden_postprocess.py)."""
    coords, shape = POST[name + "/coords"], tuple(int(x) for x in POST[name + "/shape"])
    ks, dil = tuple(int(x) for x in POST[name + "/ksize"]), tuple(int(x) for x in POST[name + "/dilation"])
    cache = build_cache(coords, shape, ks, dil)
    assert np.array_equal(u32(cache["neighbor_map"]), POST[name + "/neighbor_map"])
    assert np.array_equal(cache["gray_code"].cpu().numpy(), POST[name + "/gray_code"])
    for key in ("valid_signal_i", "valid_signal_o", "valid_signal_seg"):
        assert np.array_equal(u32(cache[key]), POST[f"{name}/{key}"]), key
    # equal codes may be ordered differently (the reference's argsort is unstable): same codes along both orders,
    # hence the same per-tile offset lists
    gray = POST[name + "/gray_code"]
    binary = orc.gray_binary_code(POST[name + "/neighbor_map"])[1]
    ours, theirs = cache["sorted_idx"].cpu().numpy(), POST[name + "/sorted_idx"]
    assert np.array_equal(binary[ours], binary[theirs])
    for block in (128, 32):
        assert np.array_equal(cache.valid_kernel_callback(block).cpu().numpy(), POST[f"{name}/valid_kernel_{block}"])
        assert np.array_equal(cache.valid_kernel_seg_callback(block).cpu().numpy(), POST[f"{name}/valid_kernel_seg_{block}"])


def test_meta_word_helpers(K):
    """The pooled zeroed words handed to a build are zero, disjoint and survive the pool's renewal; the word fetch brings
    device words into pinned memory on the stream."""
    from flexgemm_b200 import _cabi
    seen = []
    for _ in range(200):                       # more than one pool of 4096 words
        w = K._zeroed_words(DEV, 30)
        assert w.shape == (30,) and int(w.view(torch.int32).abs().sum().item()) == 0
        seen.append(w)
        w.view(torch.int32).fill_(7)           # a build overwrites its words; later slices must stay zero
    ptrs = sorted(t.data_ptr() for t in seen)
    assert all(b - a >= 120 for a, b in zip(ptrs, ptrs[1:]))
    src = torch.arange(30, dtype=torch.int32, device=DEV)
    dst = torch.zeros(30, dtype=torch.int32).pin_memory()
    rc = _cabi.lib().fgb_fetch_words_async(dst.data_ptr(), src.data_ptr(), 120, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert torch.equal(dst, src.cpu())
    assert _cabi.lib().fgb_fetch_words_async(0, src.data_ptr(), 8, 0) == -1
