"""GPU parity tests of the generic (strided) sparse conv: every call goes
through the C ABI and is compared with the golden fixtures made by the
reference's pure-torch code and with the CPU oracle.

Bars: coordinates, maps, masks and pair lists bit-exact; fp32 with TF32
disabled within 1e-4 relative; 16-bit features and gradients within
max|x - ref| <= 1e-2 * max|ref|."""
import os

import numpy as np
import pytest
import torch

from oracle import submconv_oracle as orc

pytestmark = pytest.mark.gpu

GOLD = os.path.join(os.path.dirname(__file__), "golden")
SP = np.load(os.path.join(GOLD, "sparse_conv.npz"))
TAGS = sorted({k.rsplit(".", 1)[0] for k in SP.files})
DEV = torch.device("cuda:0")


@pytest.fixture(autouse=True)
def _defaults():
    from flexgemm_b200.kernels import config
    from flexgemm_b200.ops import spconv
    spconv.set_algorithm(spconv.Algorithm.MASKED_IMPLICIT_GEMM_SPLITK)
    spconv.set_hashmap_ratio(2.0)
    spconv.SERIALIZATION_MODE = spconv.SerializationMode.BXYZ
    config.allow_tf32 = True
    yield
    config.allow_tf32 = True
    spconv.SERIALIZATION_MODE = spconv.SerializationMode.BXYZ


def u32(t):
    return t.detach().cpu().view(torch.int32).numpy().view(np.uint32)


def geom_of(tag):
    g = tuple(int(v) for v in SP[tag + ".geom"])
    return g[0:3], g[3:6], g[6:9], g[9:12]


def dev_coords(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def rel_err(a, b):
    a, b = a.detach().double().cpu(), b.detach().double().cpu()
    return ((a - b).abs().max() / b.abs().max().clamp_min(1e-30)).item()


def check_sparse_cache(cache, nbr, bwd, V):
    """Everything derived from the maps, against the oracle's definitions."""
    assert np.array_equal(u32(cache["neighbor_map"]), nbr)
    assert np.array_equal(u32(cache["neighbor_map_bwd"]), bwd)
    gray, binary = orc.gray_binary_code(nbr)
    assert np.array_equal(cache["gray_code"].cpu().numpy(), gray)
    assert orc.is_valid_sorted_idx(cache["sorted_idx"].cpu().numpy(), binary)
    vi, vo, seg = orc.valid_signal(nbr)
    assert np.array_equal(u32(cache["valid_signal_seg"]), seg)
    assert np.array_equal(u32(cache["valid_signal_i"]), vi)
    assert np.array_equal(u32(cache["valid_signal_o"]), vo)
    cache._ensure_bwd_order()
    gray_b, binary_b = orc.gray_binary_code(bwd)
    assert np.array_equal(cache["gray_code_bwd"].cpu().numpy(), gray_b)
    assert orc.is_valid_sorted_idx(cache["sorted_idx_bwd"].cpu().numpy(), binary_b)
    for B in (128, 32):
        vk, vseg = orc.valid_kernel(gray, cache["sorted_idx"].cpu().numpy(), B)
        assert np.array_equal(cache.valid_kernel_callback(B).cpu().numpy(), vk)
        assert np.array_equal(cache.valid_kernel_seg_callback(B).cpu().numpy(), vseg)
        vk, vseg = orc.valid_kernel(gray_b, cache["sorted_idx_bwd"].cpu().numpy(), B)
        assert np.array_equal(cache.valid_kernel_bwd_callback(B).cpu().numpy(), vk)
        assert np.array_equal(cache.valid_kernel_bwd_seg_callback(B).cpu().numpy(), vseg)


@pytest.mark.parametrize("tag", TAGS)
def test_out_coords_and_maps_match_golden(tag):
    from flexgemm_b200.ops.spconv import SparseConv3dFunction as F
    coords, shape = dev_coords(SP[tag + ".coords"]), torch.Size([int(v) for v in SP[tag + ".shape"]])
    k, s, p, d = geom_of(tag)
    oc = F._get_output_coords(coords, shape, k, s, p, d)
    assert oc.dtype == torch.int32 and oc.is_contiguous()
    assert np.array_equal(oc.cpu().numpy(), SP[tag + ".out_coords"])
    assert np.array_equal(F._get_output_coords_torch(coords, shape, k, s, p, d).cpu().numpy(), SP[tag + ".out_coords"])
    if tag + ".nbr" not in SP.files:
        return
    cache = F._compute_neighbor_cache(coords, oc, shape, k, s, p, d, True)
    check_sparse_cache(cache, SP[tag + ".nbr"], SP[tag + ".nbr_bwd"], k[0] * k[1] * k[2])
    inf = F._compute_neighbor_cache(coords, oc, shape, k, s, p, d, False)
    assert inf["neighbor_map_bwd"] is None and np.array_equal(u32(inf["neighbor_map"]), SP[tag + ".nbr"])
    assert int(inf["build_status"].item()) == 0


@pytest.mark.parametrize("tag", [t for t in TAGS if t + ".out" in SP.files])
def test_conv_matches_golden_fp32(tag):
    """fp32 with TF32 disabled against the reference's explicit path: <= 1e-4 relative."""
    from flexgemm_b200.kernels import config
    from flexgemm_b200.ops.spconv import sparse_conv3d
    config.allow_tf32 = False
    coords, shape = dev_coords(SP[tag + ".coords"]), torch.Size([int(v) for v in SP[tag + ".shape"]])
    k, s, p, d = geom_of(tag)
    feats = torch.from_numpy(SP[tag + ".feats"]).to(DEV).requires_grad_(True)
    weight = torch.from_numpy(SP[tag + ".weight"]).to(DEV).requires_grad_(True)
    bias = torch.from_numpy(SP[tag + ".bias"]).to(DEV).requires_grad_(True)
    out, oc, cache = sparse_conv3d(feats, coords, shape, weight, bias, stride=s, padding=p, dilation=d)
    assert np.array_equal(oc.cpu().numpy(), SP[tag + ".out_coords"])
    out.backward(torch.from_numpy(SP[tag + ".gout"]).to(DEV))
    assert rel_err(out, torch.from_numpy(SP[tag + ".out"])) <= 1e-4
    assert rel_err(feats.grad, torch.from_numpy(SP[tag + ".gin"])) <= 1e-4
    assert rel_err(weight.grad, torch.from_numpy(SP[tag + ".gw"])) <= 1e-4
    assert rel_err(bias.grad, torch.from_numpy(SP[tag + ".gb"])) <= 1e-4


GEOMS = {
    "down_k2s2": ((2, 2, 2), (2, 2, 2), (0, 0, 0), (1, 1, 1)),
    "down_k3s2p1": ((3, 3, 3), (2, 2, 2), (1, 1, 1), (1, 1, 1)),
    "same_k3s1p1": ((3, 3, 3), (1, 1, 1), (1, 1, 1), (1, 1, 1)),
}


@pytest.mark.parametrize("gname", sorted(GEOMS))
@pytest.mark.parametrize("dtype,ci,co", [(torch.float16, 64, 128), (torch.bfloat16, 256, 64), (torch.float32, 32, 32)])
def test_conv_matches_oracle(gname, dtype, ci, co):
    """RES=48 shell, two samples: forward and all gradients against the oracle
    evaluated in fp64 on the same (rounded) inputs."""
    from flexgemm_b200.ops.spconv import sparse_conv3d
    k, s, p, d = GEOMS[gname]
    res = 48
    coords_np = orc.shell_coords(res, batch=2, scales=(1.0, 0.8))
    shape = (2, ci, res, res, res)
    g = torch.Generator().manual_seed(5)
    V = k[0] * k[1] * k[2]
    feats = torch.randn(coords_np.shape[0], ci, generator=g).to(dtype)
    weight = (torch.randn(co, *k, ci, generator=g) / (V * ci) ** 0.5).to(dtype)
    bias = torch.randn(co, generator=g).to(dtype)
    oc_ref = orc.sparse_out_coords(coords_np, shape, k, s, p, d)
    nbr, bwd = orc.sparse_neighbor_maps(coords_np, oc_ref, shape, k, s, p, d)
    gout = torch.randn(oc_ref.shape[0], co, generator=g).to(dtype)
    ref_out = orc.conv_forward(feats.double(), nbr, weight.double(), bias.double())
    ref_gin, ref_gw, ref_gb = orc.sparse_conv_backward(gout.double(), feats.double(), nbr, bwd, weight.double())

    f = feats.to(DEV).requires_grad_(True)
    w = weight.to(DEV).requires_grad_(True)
    b = bias.to(DEV).requires_grad_(True)
    out, oc, cache = sparse_conv3d(f, dev_coords(coords_np), torch.Size(shape), w, b, stride=s, padding=p, dilation=d)
    assert np.array_equal(oc.cpu().numpy(), oc_ref)
    assert np.array_equal(u32(cache["neighbor_map"]), nbr) and np.array_equal(u32(cache["neighbor_map_bwd"]), bwd)
    out.backward(gout.to(DEV))
    tol = 1e-2
    assert rel_err(out, ref_out) <= tol
    assert rel_err(f.grad, ref_gin) <= tol
    assert rel_err(w.grad, ref_gw) <= tol
    assert rel_err(b.grad, ref_gb) <= tol
    # a second call with the cache and the coordinates it was built for reproduces the output bit for bit
    out2, _, _ = sparse_conv3d(f.detach(), dev_coords(coords_np), torch.Size(shape), w.detach(), b.detach(), neighbor_cache=cache,
                               out_coords=oc, stride=s, padding=p, dilation=d)
    assert torch.equal(out2, out.detach())


def test_given_out_coords_with_isolated_voxels():
    """Caller-provided output coordinates: some have no input under the kernel
    (their output is the bias) and some inputs feed no output (zero gradient)."""
    from flexgemm_b200.ops.spconv import sparse_conv3d
    res, ci, co = 24, 32, 64
    coords_np = orc.shell_coords(res)
    shape = (1, ci, res, res, res)
    k, s, p, d = (3, 3, 3), (2, 2, 2), (1, 1, 1), (1, 1, 1)
    auto = orc.sparse_out_coords(coords_np, shape, k, s, p, d)
    rng = np.random.default_rng(2)
    keep = auto[rng.permutation(len(auto))[: len(auto) // 2]]           # unsorted half of the natural outputs
    empty = np.array([[0, 6, 6, 6], [0, 5, 6, 6], [0, 6, 5, 6]], dtype=np.int32)  # sphere centre: nothing nearby
    oc_np = np.ascontiguousarray(np.concatenate([keep[:7], empty, keep[7:]], axis=0))
    nbr, bwd = orc.sparse_neighbor_maps(coords_np, oc_np, shape, k, s, p, d)
    assert (nbr[7:10] == orc.INVALID).all() and ((bwd == orc.INVALID).all(axis=1)).any()
    g = torch.Generator().manual_seed(9)
    feats = torch.randn(coords_np.shape[0], ci, generator=g).half()
    weight = (torch.randn(co, *k, ci, generator=g) / (27 * ci) ** 0.5).half()
    bias = torch.randn(co, generator=g).half()
    gout = torch.randn(oc_np.shape[0], co, generator=g).half()
    ref_out = orc.conv_forward(feats.double(), nbr, weight.double(), bias.double())
    ref_gin, ref_gw, _ = orc.sparse_conv_backward(gout.double(), feats.double(), nbr, bwd, weight.double())
    f, w, b = feats.to(DEV).requires_grad_(True), weight.to(DEV).requires_grad_(True), bias.to(DEV).requires_grad_(True)
    out, oc, cache = sparse_conv3d(f, dev_coords(coords_np), torch.Size(shape), w, b, out_coords=dev_coords(oc_np), stride=s,
                                   padding=p, dilation=d)
    assert np.array_equal(oc.cpu().numpy(), oc_np)
    assert "sorted_idx_bwd" in cache  # given coordinates: the backward map is sorted at build time, as in the reference
    out.backward(gout.to(DEV))
    assert torch.equal(out[7:10].cpu(), bias.expand(3, co))
    assert rel_err(out, ref_out) <= 1e-2 and rel_err(f.grad, ref_gin) <= 1e-2 and rel_err(w.grad, ref_gw) <= 1e-2
    dead = torch.from_numpy((bwd == orc.INVALID).all(axis=1))
    assert dead.any() and (f.grad.cpu()[dead] == 0).all()


def test_same_padding_on_own_coords_equals_submanifold_conv():
    from flexgemm_b200.ops.spconv import sparse_conv3d, sparse_submanifold_conv3d
    coords_np, feats, weight, bias, shape = orc.make_problem(32, 64, 64, "float16", seed=3)
    c = dev_coords(coords_np)
    f, w, b = feats.to(DEV), weight.to(DEV), bias.to(DEV)
    sub, _ = sparse_submanifold_conv3d(f, c, torch.Size(shape), w, b)
    gen, oc, _ = sparse_conv3d(f, c, torch.Size(shape), w, b, out_coords=c, padding=(1, 1, 1))
    assert torch.equal(gen, sub)


@pytest.mark.parametrize("mode", [1, 2])
def test_serialised_output_order(mode):
    from flexgemm_b200.ops import spconv
    from flexgemm_b200.ops.spconv import SparseConv3dFunction as F
    spconv.SERIALIZATION_MODE = mode
    coords_np = orc.shell_coords(40, batch=3, scales=(1.0, 0.7, 0.9))
    shape = (3, 0, 40, 40, 40)
    for geom in GEOMS.values():
        got = F._get_output_coords(dev_coords(coords_np), torch.Size(shape), *geom).cpu().numpy()
        assert np.array_equal(got, orc.sparse_out_coords(coords_np, shape, *geom, mode=mode))


def test_all_algorithms_agree_and_explicit_path_runs_on_gpu():
    from flexgemm_b200.ops import spconv
    from flexgemm_b200.ops.spconv import sparse_conv3d
    coords_np = orc.shell_coords(24)
    shape = torch.Size((1, 32, 24, 24, 24))
    g = torch.Generator().manual_seed(4)
    feats = torch.randn(coords_np.shape[0], 32, generator=g).half().to(DEV)
    weight = (torch.randn(32, 3, 3, 3, 32, generator=g) / 30).half().to(DEV)
    outs = {}
    for algo in spconv._ALL_ALGORITHMS:
        spconv.set_algorithm(algo)
        f, w = feats.clone().requires_grad_(True), weight.clone().requires_grad_(True)
        out, oc, _ = sparse_conv3d(f, dev_coords(coords_np), shape, w, None, stride=(2, 2, 2), padding=(1, 1, 1))
        out.float().sum().backward()
        outs[algo] = (out.detach(), f.grad, w.grad)
    base = outs[spconv.Algorithm.MASKED_IMPLICIT_GEMM_SPLITK]
    for algo, got in outs.items():
        if algo == spconv.Algorithm.EXPLICIT_GEMM:
            assert all(rel_err(a, b) <= 1e-2 for a, b in zip(got, base))
        else:
            assert all(torch.equal(a, b) for a, b in zip(got, base))


def test_downsample_res256():
    """The stride-2 conv that follows the benchmark's RES=256 shell: output set,
    both maps and the output rows at sampled positions, against the oracle."""
    from flexgemm_b200.ops.spconv import sparse_conv3d
    res, ci, co = 256, 64, 128
    coords_np = orc.shell_coords(res)
    shape = (1, ci, res, res, res)
    k, s, p, d = (2, 2, 2), (2, 2, 2), (0, 0, 0), (1, 1, 1)
    oc_ref = orc.sparse_out_coords(coords_np, shape, k, s, p, d)
    nbr, bwd = orc.sparse_neighbor_maps(coords_np, oc_ref, shape, k, s, p, d)
    g = torch.Generator().manual_seed(6)
    feats = torch.randn(coords_np.shape[0], ci, generator=g).half()
    weight = (torch.randn(co, *k, ci, generator=g) / (8 * ci) ** 0.5).half()
    f, w = feats.to(DEV).requires_grad_(True), weight.to(DEV).requires_grad_(True)
    out, oc, cache = sparse_conv3d(f, dev_coords(coords_np), torch.Size(shape), w, None, stride=s)
    assert np.array_equal(oc.cpu().numpy(), oc_ref)
    assert np.array_equal(u32(cache["neighbor_map"]), nbr) and np.array_equal(u32(cache["neighbor_map_bwd"]), bwd)
    out.float().sum().backward()
    rows = np.random.default_rng(0).choice(oc_ref.shape[0], 4000, replace=False)
    ref = orc.conv_forward(feats.double(), nbr[rows], weight.double())
    assert rel_err(out[torch.from_numpy(rows).to(DEV)], ref) <= 1e-2
    rows_in = np.random.default_rng(1).choice(coords_np.shape[0], 4000, replace=False)
    ones = torch.ones(oc_ref.shape[0], co, dtype=torch.float64)
    col = orc._im2col(ones, torch.from_numpy(bwd[rows_in].astype(np.int64)), 8)
    ref_gin = torch.mm(col, weight.double().reshape(co, 8, ci).transpose(0, 1).reshape(8 * co, ci))
    assert rel_err(f.grad[torch.from_numpy(rows_in).to(DEV)], ref_gin) <= 1e-2
