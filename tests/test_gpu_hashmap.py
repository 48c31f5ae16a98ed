"""The generic hash map with caller-chosen values, in the reference's own
layout and call shapes: insert followed by lookup returns the inserted values
for every key / value width (the reference's round-trip test,
tests/hashmap.py:8-88 in its tree), absent keys give all ones, a table without
room reports instead of spinning."""
import numpy as np
import pytest
import torch

from oracle import submconv_oracle as orc

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")

WIDTHS = [(torch.uint32, torch.uint32), (torch.uint32, torch.uint64), (torch.uint64, torch.uint32), (torch.uint64, torch.uint64)]


def as_int64(t):
    return t.cpu().view(torch.int32 if t.dtype == torch.uint32 else torch.int64).to(torch.int64)


@pytest.mark.parametrize("res", [1, 2, 8, 32, 64])
@pytest.mark.parametrize("kdt,vdt", WIDTHS)
def test_insert_3d_then_lookup_3d_round_trip(res, kdt, vdt):
    from flexgemm_b200.kernels import cuda as K
    coords_np = orc.reference_sphere_coords(res)
    coords = torch.from_numpy(coords_np).to(DEV)
    n = coords.shape[0]
    hashmap_keys = torch.full((2 * n,), torch.iinfo(kdt).max, dtype=kdt, device=DEV)
    hashmap_values = torch.empty((2 * n,), dtype=vdt, device=DEV)
    values = torch.randint(0, 2 ** 31 - 1, (n,), device=DEV).to(vdt)
    K.hashmap_insert_3d(hashmap_keys, hashmap_values, coords, values, res, res, res)
    got = K.hashmap_lookup_3d(hashmap_keys, hashmap_values, coords, res, res, res)
    assert got.dtype == vdt
    assert torch.equal(as_int64(got), as_int64(values))
    # voxels that were not inserted, and coordinates outside the grid, are absent
    miss = coords.clone()
    miss[:, 1] = res + 3
    absent = K.hashmap_lookup_3d(hashmap_keys, hashmap_values, miss, res, res, res)
    assert bool((as_int64(absent) == -1).all())


@pytest.mark.parametrize("kdt,vdt", WIDTHS)
def test_insert_then_lookup_by_key(kdt, vdt):
    from flexgemm_b200.kernels import cuda as K
    rng = np.random.default_rng(3)
    n = 50_000
    hi = 2 ** 31 - 2 if kdt == torch.uint32 else 2 ** 62
    raw = np.unique(rng.integers(0, hi, size=2 * n, dtype=np.int64))[:n]
    rng.shuffle(raw)
    keys = torch.from_numpy(raw).to(DEV).to(kdt)
    values = torch.arange(raw.size, device=DEV).to(vdt)
    hashmap_keys = torch.full((2 * raw.size,), torch.iinfo(kdt).max, dtype=kdt, device=DEV)
    hashmap_values = torch.empty_like(hashmap_keys, dtype=vdt)
    K.hashmap_insert(hashmap_keys, hashmap_values, keys, values)
    assert torch.equal(as_int64(K.hashmap_lookup(hashmap_keys, hashmap_values, keys)), as_int64(values))
    others = torch.from_numpy(raw + 1).to(DEV).to(kdt)          # raw + 1 may collide with a present key: check against the set
    got = as_int64(K.hashmap_lookup(hashmap_keys, hashmap_values, others)).numpy()
    present = np.isin(raw + 1, raw)
    assert (got[~present] == -1).all()
    pos = {int(k): i for i, k in enumerate(raw)}
    assert all(got[i] == pos[int(raw[i] + 1)] for i in np.nonzero(present)[0])
    with pytest.raises(RuntimeError, match="Keys must be"):
        K.hashmap_lookup(hashmap_keys, hashmap_values, keys.to(torch.uint64 if kdt == torch.uint32 else torch.uint32))


def test_idx_as_val_matches_the_neighbor_map_of_the_oracle():
    """insert_3d_idx_as_val + lookup_3d of the 27 shifted coordinate sets rebuilds the neighbour map."""
    from flexgemm_b200.kernels import cuda as K
    from flexgemm_b200.ops import utils
    res = 24
    coords_np = orc.shell_coords(res)
    shape = (1, 8, res, res, res)
    coords = torch.from_numpy(coords_np).to(DEV)
    hashmap_keys, hashmap_values = utils.init_hashmap(shape, 2 * coords.shape[0], DEV)
    assert hashmap_keys.dtype == torch.uint32 and hashmap_values.dtype == torch.uint32
    assert utils.init_hashmap((8, 1, 1024, 1024, 1024), 16, DEV, with_values=False).dtype == torch.uint64
    K.hashmap_insert_3d_idx_as_val(hashmap_keys, hashmap_values, coords, res, res, res)
    want = orc.neighbor_map(coords_np, shape)
    v = 0
    for dx in (-1, 0, 1):
        for dy in (-1, 0, 1):
            for dz in (-1, 0, 1):
                q = coords.clone()
                q[:, 1] += dx
                q[:, 2] += dy
                q[:, 3] += dz
                got = K.hashmap_lookup_3d(hashmap_keys, hashmap_values, q, res, res, res)
                assert np.array_equal(got.cpu().view(torch.int32).numpy().view(np.uint32), want[:, v]), v
                v += 1


def test_full_table_is_reported():
    from flexgemm_b200.kernels import cuda as K
    n = 1000
    keys = torch.arange(n, device=DEV).to(torch.uint32)
    hashmap_keys = torch.full((n // 2,), torch.iinfo(torch.uint32).max, dtype=torch.uint32, device=DEV)
    hashmap_values = torch.empty_like(hashmap_keys)
    with pytest.raises(RuntimeError, match="hash table full"):
        K.hashmap_insert(hashmap_keys, hashmap_values, keys, keys)
