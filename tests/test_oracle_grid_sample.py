"""The grid-sample oracle and the package's library-only helper against golden
vectors produced by the reference's own torch path
(tests/golden/make_golden_grid_sample.py)."""
import os

import numpy as np
import pytest
import torch

from oracle import submconv_oracle as orc

GS = np.load(os.path.join(os.path.dirname(__file__), "golden", "grid_sample.npz"))
NAMES = sorted({k.split(".")[0] for k in GS.files})


@pytest.mark.parametrize("mode", ["nearest", "trilinear"])
@pytest.mark.parametrize("name", NAMES)
def test_oracle_matches_reference(name, mode):
    feats = torch.from_numpy(GS[name + ".feats"])
    got = orc.grid_sample(feats, GS[name + ".coords"], tuple(GS[name + ".shape"]), GS[name + ".query"], mode)
    want = torch.from_numpy(GS[f"{name}.{mode}"])
    assert got.shape == want.shape
    if mode == "nearest":
        assert torch.equal(got, want)
    else:
        assert (got - want).abs().max() <= 1e-6 * want.abs().max()
    # the fixture exercises both outcomes
    hit = want.abs().sum(-1) > 0
    assert hit.any() and (~hit).any()


@pytest.mark.parametrize("mode", ["nearest", "trilinear"])
@pytest.mark.parametrize("name", NAMES)
def test_package_torch_helper_matches_reference(name, mode):
    from flexgemm_b200.ops.grid_sample import grid_sample_3d_torch
    feats = torch.from_numpy(GS[name + ".feats"])
    coords = torch.from_numpy(GS[name + ".coords"])
    got = grid_sample_3d_torch(feats, coords, torch.Size([int(v) for v in GS[name + ".shape"]]), torch.from_numpy(GS[name + ".query"]), mode)
    want = torch.from_numpy(GS[f"{name}.{mode}"])
    assert (got - want).abs().max() <= 1e-6 * want.abs().max()


def test_weights_are_normalised_over_existing_voxels():
    coords = np.array([[0, 2, 2, 2], [0, 3, 2, 2]], dtype=np.int32)
    shape = (1, 4, 6, 6, 6)
    q = np.array([[[3.0, 2.5, 2.5], [2.5, 2.5, 2.5], [0.2, 0.2, 0.2]]], dtype=np.float32)
    rows, w = orc.grid_sample_maps(coords, shape, q, True)
    assert np.allclose(w[0, 0].sum(), 1.0) and sorted(rows[0, 0][rows[0, 0] >= 0].tolist()) == [0, 1]
    assert np.allclose(w[0, 0][rows[0, 0] >= 0], 0.5)            # half way between the two voxel centres
    assert np.allclose(w[0, 1].sum(), 1.0) and np.allclose(np.sort(w[0, 1])[-2:], [0.0, 1.0])   # exactly on the first voxel's centre: the second voxel is a corner with weight 0
    assert (rows[0, 2] < 0).all() and np.all(w[0, 2] == 0)        # nothing around: zero output
    g = orc.grid_sample_backward(torch.ones(1, 3, 4), coords, shape, q, "trilinear")
    assert torch.allclose(g.sum(), torch.tensor(8.0, dtype=torch.float64))   # two points with unit weight, four channels
