"""The CPU oracle against golden vectors produced by the reference's own
pure-torch implementation (tests/golden/make_golden.py)."""
import os

import numpy as np
import pytest
import torch

from oracle import submconv_oracle as orc

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def _cases(npz):
    return sorted({k.split("/")[0] for k in npz.files})


MAPS = np.load(os.path.join(GOLD, "neighbor_maps.npz"))
CONV = np.load(os.path.join(GOLD, "conv_explicit.npz"))


@pytest.mark.parametrize("name", _cases(MAPS))
def test_neighbor_map_matches_reference(name):
    coords = MAPS[name + "/coords"]
    got = orc.neighbor_map(coords, MAPS[name + "/shape"], tuple(MAPS[name + "/ksize"]), tuple(MAPS[name + "/dilation"]))
    assert got.dtype == np.uint32
    assert np.array_equal(got, MAPS[name + "/neighbor_map"])


@pytest.mark.parametrize("name", _cases(CONV))
def test_explicit_conv_matches_reference(name):
    t = {k: torch.from_numpy(CONV[f"{name}/{k}"]) for k in
         ("coords", "feats", "weight", "bias", "out", "grad_out", "grad_feats", "grad_weight", "grad_bias")}
    nbr = orc.neighbor_map(t["coords"].numpy(), CONV[name + "/shape"])
    out = orc.conv_forward(t["feats"], nbr, t["weight"], t["bias"])
    gin, gw, gb = orc.conv_backward(t["grad_out"], t["feats"], nbr, t["weight"])
    # same operations in the same order on the same library: bit-exact
    assert torch.equal(out, t["out"])
    assert torch.equal(gin, t["grad_feats"])
    assert torch.equal(gw, t["grad_weight"])
    assert torch.equal(gb, t["grad_bias"])


def test_explicit_conv_matches_dense_conv3d():
    """Independent check of the offset/axis conventions: the sparse result equals
    a dense conv3d with weight.permute(0,4,1,2,3) sampled at the active voxels."""
    coords, feats, weight, bias, shape = orc.make_problem(8, 5, 7, "float64", seed=3, batch=2)
    nbr = orc.neighbor_map(coords.numpy(), shape)
    out = orc.conv_forward(feats, nbr, weight, bias)
    B, C, W, H, D = shape
    dense = torch.zeros(B, C, W, H, D, dtype=feats.dtype)
    c = coords.long()
    dense[c[:, 0], :, c[:, 1], c[:, 2], c[:, 3]] = feats
    ref = torch.nn.functional.conv3d(dense, weight.permute(0, 4, 1, 2, 3), bias, padding=1)
    ref = ref[c[:, 0], :, c[:, 1], c[:, 2], c[:, 3]]
    assert torch.allclose(out, ref, atol=1e-12)


def test_map_symmetry_and_center():
    coords = orc.shell_coords(16, batch=2, scales=(1.0, 0.7))
    nbr = orc.neighbor_map(coords, (2, 0, 16, 16, 16))
    n, V = nbr.shape
    assert np.array_equal(nbr[:, V // 2], np.arange(n, dtype=np.uint32))
    rows, vs = np.nonzero(nbr != orc.INVALID)
    assert np.array_equal(nbr[nbr[rows, vs], V - 1 - vs], rows.astype(np.uint32))


def test_postprocess_definitions():
    coords = orc.shell_coords(16)
    cache = orc.neighbor_cache(coords, (1, 0, 16, 16, 16))
    nbr, gray, binary = cache["neighbor_map"], cache["gray_code"], cache["binary_code"]
    n, V = nbr.shape
    # gray bit v <=> valid; binary is the prefix-xor decode
    for v in range(V):
        assert np.array_equal((gray >> v) & 1, (nbr[:, v] != orc.INVALID).astype(np.int32))
    g = gray.view(np.uint32)
    assert np.array_equal((binary.view(np.uint32) ^ (binary.view(np.uint32) >> 1)) & ((1 << V) - 1), g)
    assert orc.is_valid_sorted_idx(cache["sorted_idx"], binary)
    assert not orc.is_valid_sorted_idx(cache["sorted_idx"][::-1].copy(), binary) or n < 2
    vs_i, vs_o, seg = cache["valid_signal_i"], cache["valid_signal_o"], cache["valid_signal_seg"]
    assert seg[0] == 0 and seg[-1] == orc.useful_pairs(nbr) == vs_i.shape[0]
    for v in range(V):
        o = vs_o[seg[v]:seg[v + 1]]
        assert np.all(np.diff(o.astype(np.int64)) > 0)
        assert np.array_equal(nbr[o, v], vs_i[seg[v]:seg[v + 1]])
    for block in (16, 64, 128):
        vk, vseg = orc.valid_kernel(gray, cache["sorted_idx"], block)
        masks = orc.tile_masks(gray, cache["sorted_idx"], block)
        assert vseg[-1] == vk.shape[0] == sum(bin(int(m)).count("1") for m in masks)
        # independent of tie order: a different valid argsort gives the same lists
        alt = np.lexsort((-np.arange(n), binary)).astype(np.int64)
        assert orc.is_valid_sorted_idx(alt, binary)
        vk2, vseg2 = orc.valid_kernel(gray, alt, block)
        assert np.array_equal(vk, vk2) and np.array_equal(vseg, vseg2)


def test_workload_sizes():
    """Voxel and pair counts of the benchmark shells (float32 distance rule)."""
    c = orc.shell_coords(32)
    assert c.shape[0] == 2520
    assert orc.useful_pairs(orc.neighbor_map(c, (1, 0, 32, 32, 32))) == 27528
    c = orc.shell_coords(64)
    assert c.shape[0] == 9968


def test_empty_input():
    nbr = orc.neighbor_map(np.zeros((0, 4), np.int32), (1, 0, 4, 4, 4))
    assert nbr.shape == (0, 27)
    gray, binary = orc.gray_binary_code(nbr)
    assert gray.shape == (0,)
    vs_i, vs_o, seg = orc.valid_signal(nbr)
    assert vs_i.shape == (0,) and np.array_equal(seg, np.zeros(28, np.uint32))


def test_residual_block_epilogue_is_the_torch_sequence():
    """The oracle's epilogue equals what a caller of the reference runs between
    convs with torch kernels, rounding included (SiLU to one unit in the last place); its SiLU derivative equals autograd's."""
    g = torch.Generator().manual_seed(0)
    y32 = torch.randn(257, 40, generator=g) * 3
    res32 = torch.randn(257, 40, generator=g)
    for dt in (torch.float16, torch.bfloat16, torch.float32):
        y, res = y32.to(dt), res32.to(dt)
        want = torch.nn.functional.silu(y) + res
        got = orc.residual_block_epilogue(y.float(), "silu", res.float(), dt).to(dt)
        # torch's silu may round its fp32 intermediate differently: one unit in the last place of the type at most
        assert torch.allclose(got.double(), want.double(), rtol=2 * torch.finfo(dt).eps, atol=1e-6), dt
        assert torch.equal(orc.residual_block_epilogue(y.float(), None, res.float(), dt).to(dt), y + res)
    yd = y32.double().requires_grad_(True)
    gout = res32.double()
    torch.nn.functional.silu(yd).backward(gout)
    assert torch.allclose(orc.silu_backward(y32.double(), gout), yd.grad, rtol=1e-12, atol=1e-12)
    with pytest.raises(ValueError):
        orc.residual_block_epilogue(y32, "gelu")


# ----------------------------------------------------------------------------
# the derived cache tensors against outputs of the reference's own CUDA functions
# ----------------------------------------------------------------------------
POST = np.load(os.path.join(GOLD, "postprocess.npz"))


@pytest.mark.parametrize("name", sorted({k.split("/")[0] for k in POST.files}))
def test_postprocessing_restatement_matches_reference_cuda_output(name):
    """gray code, pair lists, segment table and per-tile valid-offset lists as the reference's
    compiled hashmap_build_submanifold_conv_neighbour_map /
    neighbor_map_post_process_for_masked_implicit_gemm_{1,2} produced them on a GPU
    (fixture made by tests/golden/make_golden_postprocess.py): bit-exact, and the dtypes too.
    sorted_idx comes from an unstable argsort there, so it is checked as a property and
    the valid-offset lists are derived from the reference's own permutation."""
    coords, shape = POST[name + "/coords"], tuple(int(x) for x in POST[name + "/shape"])
    ks, dil = tuple(int(x) for x in POST[name + "/ksize"]), tuple(int(x) for x in POST[name + "/dilation"])
    ours = orc.neighbor_cache(coords, shape, ks, dil)
    for key in ("neighbor_map", "gray_code", "valid_signal_i", "valid_signal_o", "valid_signal_seg"):
        assert ours[key].dtype == POST[f"{name}/{key}"].dtype, key
        assert np.array_equal(ours[key], POST[f"{name}/{key}"]), key
    sidx = POST[name + "/sorted_idx"]
    assert sidx.dtype == np.int64
    assert orc.is_valid_sorted_idx(sidx, ours["binary_code"])
    for block in (128, 32):
        vk, seg = orc.valid_kernel(ours["gray_code"], sidx, block)
        assert vk.dtype == POST[f"{name}/valid_kernel_{block}"].dtype and seg.dtype == POST[f"{name}/valid_kernel_seg_{block}"].dtype
        assert np.array_equal(vk, POST[f"{name}/valid_kernel_{block}"])
        assert np.array_equal(seg, POST[f"{name}/valid_kernel_seg_{block}"])
