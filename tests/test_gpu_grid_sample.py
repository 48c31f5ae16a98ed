"""GPU parity tests of the generic table calls and the sparse grid sample.

Bars: rows of the neighbour maps bit-exact against the oracle; trilinear weights
within 1e-6; fp32 features within 1e-5 relative of the reference's golden
vectors; 16-bit features and all gradients within 1e-2 * max|ref|."""
import os

import numpy as np
import pytest
import torch

from oracle import submconv_oracle as orc

pytestmark = pytest.mark.gpu

GS = np.load(os.path.join(os.path.dirname(__file__), "golden", "grid_sample.npz"))
NAMES = sorted({k.split(".")[0] for k in GS.files})
DEV = torch.device("cuda:0")


def u32(t):
    return t.detach().cpu().view(torch.int32).numpy().view(np.uint32)


def rel_err(a, b):
    a, b = a.detach().double().cpu(), b.detach().double().cpu()
    return ((a - b).abs().max() / b.abs().max().clamp_min(1e-30)).item()


def build_table(coords_np, shape):
    from flexgemm_b200.kernels import cuda as K
    from flexgemm_b200.ops import utils
    coords = torch.from_numpy(np.ascontiguousarray(coords_np)).to(DEV)
    slots = max(2 * coords.shape[0], 1)
    table, key_bits = utils.init_table(shape, slots, DEV)
    status = K.table_insert_3d_idx_as_val(table, key_bits, slots, coords, *[int(v) for v in shape[-3:]])
    assert int(status.item()) == 0
    return table, key_bits, slots


@pytest.mark.parametrize("name", NAMES)
def test_table_lookup_and_neighbor_maps(name):
    from flexgemm_b200.kernels import cuda as K
    coords, shape, q = GS[name + ".coords"], tuple(int(v) for v in GS[name + ".shape"]), GS[name + ".query"]
    W, H, D = shape[-3:]
    table, key_bits, slots = build_table(coords, shape)
    # plain lookups: every stored voxel, its +x neighbour, and points outside the grid
    probe = np.concatenate([coords, coords + np.array([0, 1, 0, 0], dtype=np.int32), np.array([[0, -1, 0, 0], [0, 0, H, 0]], dtype=np.int32)])
    got = u32(K.table_lookup_3d(table, key_bits, slots, torch.from_numpy(np.ascontiguousarray(probe)).to(DEV), W, H, D))
    want = orc._rows_of(coords, shape, probe.astype(np.int64))
    assert np.array_equal(got, np.where(want < 0, 0xFFFFFFFF, want).astype(np.uint32))
    qd = torch.from_numpy(q).to(DEV)
    nb = u32(K.grid_sample_neighbor_map(table, key_bits, slots, qd, W, H, D, False))
    rows = orc.grid_sample_maps(coords, shape, q, False)
    assert np.array_equal(nb, np.where(rows < 0, 0xFFFFFFFF, rows).astype(np.uint32))
    nb8, w8 = K.grid_sample_neighbor_map(table, key_bits, slots, qd, W, H, D, True)
    rows8, ww = orc.grid_sample_maps(coords, shape, q, True)
    assert np.array_equal(u32(nb8), np.where(rows8 < 0, 0xFFFFFFFF, rows8).astype(np.uint32))
    assert np.abs(w8.cpu().numpy() - ww).max() <= 1e-6


@pytest.mark.parametrize("mode", ["nearest", "trilinear"])
@pytest.mark.parametrize("name", NAMES)
def test_grid_sample_matches_golden_fp32(name, mode):
    from flexgemm_b200.ops.grid_sample import grid_sample_3d, grid_sample_3d_torch
    shape = torch.Size([int(v) for v in GS[name + ".shape"]])
    feats = torch.from_numpy(GS[name + ".feats"]).to(DEV).requires_grad_(True)
    coords = torch.from_numpy(GS[name + ".coords"]).to(DEV)
    q = torch.from_numpy(GS[name + ".query"]).to(DEV)
    out = grid_sample_3d(feats, coords, shape, q, mode)
    want = torch.from_numpy(GS[f"{name}.{mode}"])
    assert rel_err(out, want) <= 1e-5
    assert rel_err(grid_sample_3d_torch(feats.detach(), coords, shape, q, mode), want) <= 1e-5   # the library-only helper on the GPU
    g = torch.Generator().manual_seed(3)
    gout = torch.randn(out.shape, generator=g)
    out.backward(gout.to(DEV))
    ref = orc.grid_sample_backward(gout, GS[name + ".coords"], tuple(shape), GS[name + ".query"], mode)
    assert rel_err(feats.grad, ref) <= 1e-5


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("mode", ["nearest", "trilinear"])
def test_grid_sample_16bit_at_scale(mode, dtype):
    """RES=128 shell, two samples, C=64, 2 x 100 000 query points near the surface."""
    from flexgemm_b200.ops.grid_sample import grid_sample_3d
    res, C, B, L = 128, 64, 2, 100_000
    coords_np = orc.shell_coords(res, batch=B, scales=(1.0, 0.7))
    shape = (B, C, res, res, res)
    g = torch.Generator().manual_seed(8)
    feats = torch.randn(coords_np.shape[0], C, generator=g).to(dtype)
    d = torch.randn(B, L, 3, generator=g)
    d = d / d.norm(dim=-1, keepdim=True)
    radius = torch.tensor([0.45 * res, 0.45 * res * 0.7]).view(B, 1, 1) - 0.5 + 0.4 * torch.randn(B, L, 1, generator=g)
    q = (d * radius + res / 2).contiguous()
    f = feats.to(DEV).requires_grad_(True)
    out = grid_sample_3d(f, torch.from_numpy(coords_np).to(DEV), torch.Size(shape), q.to(DEV), mode)
    ref = orc.grid_sample(feats.double(), coords_np, shape, q.numpy(), mode)
    assert (ref.abs().sum(-1) > 0).float().mean() > 0.5       # most points hit the shell
    assert rel_err(out, ref) <= 1e-2
    gout = torch.randn(B, L, C, generator=g).to(dtype)
    out.backward(gout.to(DEV))
    assert rel_err(f.grad, orc.grid_sample_backward(gout, coords_np, shape, q.numpy(), mode)) <= 1e-2


def test_grid_sample_64bit_keys_and_empty_inputs():
    from flexgemm_b200.ops.grid_sample import grid_sample_3d
    base = orc.shell_coords(12)
    coords_np = base.copy()
    coords_np[:, 0] = 7
    coords_np[:, 1:] += 2048 - 12
    shape = (8, 4, 2048, 2048, 2048)                          # 8 * 2048^3 = 2^36 keys
    g = torch.Generator().manual_seed(4)
    feats = torch.randn(len(coords_np), 4, generator=g)
    q = torch.zeros(8, 50, 3)
    q[7] = torch.from_numpy(coords_np[:50, 1:]).float() + torch.rand(50, 3, generator=g)
    out = grid_sample_3d(feats.to(DEV), torch.from_numpy(coords_np).to(DEV), torch.Size(shape), q.to(DEV), "trilinear")
    ref = orc.grid_sample(feats, coords_np, shape, q.numpy(), "trilinear")
    assert rel_err(out, ref) <= 1e-5 and float(out[:7].abs().max()) == 0.0
    none = grid_sample_3d(feats.to(DEV), torch.from_numpy(coords_np).to(DEV), torch.Size(shape), torch.zeros(8, 0, 3, device=DEV), "nearest")
    assert none.shape == (8, 0, 4)
