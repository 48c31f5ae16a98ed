"""The CPU oracle of the generic sparse conv against golden vectors produced by
the reference's own pure-torch implementation (tests/golden/make_golden_sparse.py)
and by its serialisation headers (tests/golden/make_golden_serialize.py)."""
import os

import numpy as np
import pytest
import torch

from oracle import submconv_oracle as orc

GOLD = os.path.join(os.path.dirname(__file__), "golden")
SP = np.load(os.path.join(GOLD, "sparse_conv.npz"))
KEYS = np.load(os.path.join(GOLD, "serialize_keys.npz"))
TAGS = sorted({k.rsplit(".", 1)[0] for k in SP.files})


def geom_of(tag):
    g = tuple(int(v) for v in SP[tag + ".geom"])
    return g[0:3], g[3:6], g[6:9], g[9:12]


@pytest.mark.parametrize("tag", TAGS)
def test_out_coords_and_maps_match_reference(tag):
    coords, shape = SP[tag + ".coords"], tuple(SP[tag + ".shape"])
    k, s, p, d = geom_of(tag)
    oc = orc.sparse_out_coords(coords, shape, k, s, p, d)
    assert oc.dtype == np.int32 and np.array_equal(oc, SP[tag + ".out_coords"])
    if tag + ".nbr" in SP.files:
        nbr, bwd = orc.sparse_neighbor_maps(coords, oc, shape, k, s, p, d)
        assert np.array_equal(nbr, SP[tag + ".nbr"])
        assert np.array_equal(bwd, SP[tag + ".nbr_bwd"])
        # the two maps describe the same set of (input, offset, output) triples
        o, v = np.nonzero(nbr != orc.INVALID)
        assert np.array_equal(bwd[nbr[o, v], v], o.astype(np.uint32))
        assert (bwd != orc.INVALID).sum() == len(o)


@pytest.mark.parametrize("tag", [t for t in TAGS if t + ".out" in SP.files])
def test_explicit_sparse_conv_matches_reference(tag):
    f, w, b, g = (torch.from_numpy(SP[tag + x]) for x in (".feats", ".weight", ".bias", ".gout"))
    nbr, bwd = SP[tag + ".nbr"], SP[tag + ".nbr_bwd"]
    out = orc.conv_forward(f, nbr, w, b)
    gin, gw, gb = orc.sparse_conv_backward(g, f, nbr, bwd, w)
    # same operations in the same order on the same library: bit-exact
    assert torch.equal(out, torch.from_numpy(SP[tag + ".out"]))
    assert torch.equal(gin, torch.from_numpy(SP[tag + ".gin"]))
    assert torch.equal(gw, torch.from_numpy(SP[tag + ".gw"]))
    assert torch.equal(gb, torch.from_numpy(SP[tag + ".gb"]))


def test_stride1_same_padding_on_own_coords_is_the_submanifold_map():
    coords = orc.shell_coords(12)
    shape = (1, 0, 12, 12, 12)
    nbr, bwd = orc.sparse_neighbor_maps(coords, coords, shape, (3, 3, 3), (1, 1, 1), (1, 1, 1), (1, 1, 1))
    sub = orc.neighbor_map(coords, shape)
    assert np.array_equal(nbr, sub)
    assert np.array_equal(bwd, sub[:, ::-1])  # the backward map is the mirrored forward map


@pytest.mark.parametrize("bits", [1, 2, 3, 5, 8, 10, 12, 21])
def test_serialisation_keys_match_reference_headers(bits):
    c = KEYS[f"bits{bits}.coords"]
    h = orc.hilbert_key(c[:, 0], c[:, 1], c[:, 2], c[:, 3], bits)
    m = orc.morton_key(c[:, 0], c[:, 1], c[:, 2], c[:, 3], bits)
    assert np.array_equal(h, KEYS[f"bits{bits}.hilbert"])
    if 3 * bits < 32:
        assert np.array_equal(m, KEYS[f"bits{bits}.morton"])
    else:
        # the reference shifts its 32-bit batch index by 3*bits >= 32 here (undefined behaviour that lands in the
        # low bits on the host): only batch 0 has a well-defined reference key
        b0 = c[:, 0] == 0
        assert b0.any() and np.array_equal(m[b0], KEYS[f"bits{bits}.morton"][b0])


def test_serialised_orders_are_permutations_of_the_bxyz_order():
    coords = orc.shell_coords(10, batch=2)
    shape = (2, 0, 10, 10, 10)
    geom = ((3, 3, 3), (2, 2, 2), (1, 1, 1), (1, 1, 1))
    base = orc.sparse_out_coords(coords, shape, *geom, mode=0)
    for mode in (1, 2):
        got = orc.sparse_out_coords(coords, shape, *geom, mode=mode)
        assert got.shape == base.shape and not np.array_equal(got, base)
        assert np.array_equal(np.unique(got, axis=0), base)
        assert np.all(np.diff(got[:, 0]) >= 0)  # batch index sits on top of the key


@pytest.mark.parametrize("tag", [t for t in TAGS if t + ".out" in SP.files])
def test_host_side_torch_path_of_the_package_matches_reference(tag):
    """The package's own library-only helpers (the torch constructions the
    reference also ships, usable without a GPU) against the golden vectors:
    output coordinates, both maps, explicit forward and backward."""
    from flexgemm_b200.ops import spconv
    from flexgemm_b200.ops.spconv import SparseConv3dFunction as F
    spconv.set_algorithm(spconv.Algorithm.EXPLICIT_GEMM)
    try:
        coords = torch.from_numpy(np.ascontiguousarray(SP[tag + ".coords"]))
        shape = torch.Size([int(v) for v in SP[tag + ".shape"]])
        k, s, p, d = geom_of(tag)
        oc = F._get_output_coords_torch(coords, shape, k, s, p, d)
        assert np.array_equal(oc.numpy(), SP[tag + ".out_coords"])
        cache = F._compute_neighbor_cache_torch(coords, oc, shape, k, s, p, d, True)
        assert np.array_equal(cache["neighbor_map"].view(torch.int32).numpy().view(np.uint32), SP[tag + ".nbr"])
        assert np.array_equal(cache["neighbor_map_bwd"].view(torch.int32).numpy().view(np.uint32), SP[tag + ".nbr_bwd"])
        f = torch.from_numpy(SP[tag + ".feats"]).requires_grad_(True)
        w = torch.from_numpy(SP[tag + ".weight"]).requires_grad_(True)
        b = torch.from_numpy(SP[tag + ".bias"]).requires_grad_(True)
        out = F._sparse_conv_forward(f, cache, w, b)
        gin, gw, gb = F._sparse_conv_backward(torch.from_numpy(SP[tag + ".gout"]), f, cache, w, b)
        for got, name in ((out, ".out"), (gin, ".gin"), (gw, ".gw"), (gb, ".gb")):
            want = torch.from_numpy(SP[tag + name])
            assert (got.detach() - want).abs().max() <= 1e-5 * want.abs().max().clamp_min(1.0)
    finally:
        spconv.set_algorithm(spconv.Algorithm.MASKED_IMPLICIT_GEMM_SPLITK)
