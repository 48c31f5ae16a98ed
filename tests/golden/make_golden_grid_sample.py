"""Generate tests/golden/grid_sample.npz from the reference's library-only grid
sample (flex_gemm/ops/grid_sample/grid_sample_torch.py:8-154).

    python tests/golden/make_golden_grid_sample.py /path/to/FlexGEMM

That code is plain torch except for two table calls into the reference's CUDA
extension, which cannot run without a GPU.  They are replaced here by an exact
dictionary (coordinate -> row, 0xffffffff where absent) -- the table has no
other observable behaviour -- so that the reference's own arithmetic (corner
enumeration, weights, normalisation, masking) produces the vectors unmodified.
"""
import importlib
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))
from oracle import submconv_oracle as orc  # noqa: E402  (input generators only)

_TABLE = {}


def _insert(keys, vals, coords, W, H, D):
    _TABLE.clear()
    for i, (b, x, y, z) in enumerate(coords.tolist()):
        _TABLE.setdefault((b, x, y, z), i)


def _lookup(keys, vals, pts, W, H, D):
    out = [_TABLE.get(tuple(p), 0xFFFFFFFF) if 0 <= p[1] < W and 0 <= p[2] < H and 0 <= p[3] < D else 0xFFFFFFFF for p in pts.tolist()]
    return torch.tensor(out, dtype=torch.int64).to(torch.uint32)


def load_reference(ref_root):
    pkg = os.path.join(ref_root, "flex_gemm")
    for name, path in (("flex_gemm", pkg), ("flex_gemm.kernels", os.path.join(pkg, "kernels")),
                       ("flex_gemm.ops", os.path.join(pkg, "ops"))):
        m = types.ModuleType(name)
        m.__path__ = [path]
        sys.modules[name] = m
    cuda = types.ModuleType("flex_gemm.kernels.cuda")
    cuda.hashmap_insert_3d_idx_as_val = _insert
    cuda.hashmap_lookup_3d = _lookup
    sys.modules["flex_gemm.kernels.cuda"] = cuda
    sys.modules["flex_gemm.kernels"].cuda = cuda
    sys.modules["flex_gemm"].kernels = sys.modules["flex_gemm.kernels"]
    sys.modules["flex_gemm"].ops = sys.modules["flex_gemm.ops"]
    importlib.import_module("flex_gemm.ops.utils")
    sys.modules["flex_gemm.ops"].utils = sys.modules["flex_gemm.ops.utils"]
    gs = types.ModuleType("flex_gemm.ops.grid_sample")
    gs.__path__ = [os.path.join(pkg, "ops", "grid_sample")]
    gs.HASHMAP_RATIO = 2.0
    sys.modules["flex_gemm.ops.grid_sample"] = gs
    sys.modules["flex_gemm.ops"].grid_sample = gs
    return importlib.import_module("flex_gemm.ops.grid_sample.grid_sample_torch")


def main():
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("FLEXGEMM_REFERENCE")
    if not ref_root:
        raise SystemExit("usage: %s <path to the FlexGEMM source tree>  (or set FLEXGEMM_REFERENCE)" % os.path.basename(__file__))
    ref = load_reference(ref_root)
    rng = np.random.default_rng(21)
    out = {}
    for name, res, batch in (("shell12", 12, 1), ("shell10b2", 10, 2)):
        coords = orc.shell_coords(res, batch=batch)
        coords = np.ascontiguousarray(coords[rng.permutation(len(coords))])   # rows in arbitrary order
        shape = (batch, 8, res, res, res)
        g = torch.Generator().manual_seed(res)
        feats = torch.randn(coords.shape[0], 8, generator=g)
        # query points: on the shell (most hit voxels), inside the grid at random, on voxel centres and faces, outside
        centre = res / 2
        theta = torch.rand(batch, 150, generator=g) * 6.2831853
        phi = (torch.rand(batch, 150, generator=g) - 0.5) * 3.1415927
        r = 0.45 * res - 0.5 + 0.3 * torch.randn(batch, 150, generator=g)
        on = torch.stack([r * torch.cos(theta) * torch.cos(phi) + centre, r * torch.sin(theta) * torch.cos(phi) + centre,
                          r * torch.sin(phi) + centre], dim=-1)
        inside = torch.rand(batch, 60, 3, generator=g) * res
        vox = torch.from_numpy(coords[rng.integers(0, len(coords), (batch, 30))][..., 1:]).float()
        exact = torch.cat([vox[:, :10] + 0.5, vox[:, 10:20], vox[:, 20:] + torch.tensor([0.5, 0.0, 1.0])], dim=1)
        outside = torch.cat([torch.rand(batch, 10, 3, generator=g) * res + res, -torch.rand(batch, 10, 3, generator=g) * 0.4], dim=1)
        pts = torch.cat([on, inside, exact, outside], dim=1).contiguous()
        c = torch.from_numpy(coords)
        out[name + ".coords"] = coords
        out[name + ".shape"] = np.array(shape, dtype=np.int64)
        out[name + ".feats"] = feats.numpy()
        out[name + ".query"] = pts.numpy()
        for mode in ("nearest", "trilinear"):
            out[f"{name}.{mode}"] = ref.grid_sample_3d_torch(feats, c, torch.Size(shape), pts, mode).numpy()
    np.savez_compressed(os.path.join(HERE, "grid_sample.npz"), **out)
    print("wrote grid_sample.npz:", {k: v.shape for k, v in out.items() if k.endswith(("nearest", "trilinear"))})


if __name__ == "__main__":
    main()
