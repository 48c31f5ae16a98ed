"""Generate tests/golden/sparse_conv.npz from the reference's own generic
sparse-conv code.

    python tests/golden/make_golden_sparse.py /path/to/FlexGEMM

As in ``make_golden.py`` only the pure-torch pieces of the reference run (its
package queries the CUDA device at import, so ``flex_gemm`` and
``flex_gemm.kernels`` are registered as empty stand-in modules first).  What is
executed, unmodified, is ``SparseConv3dFunction._get_output_coords_torch``,
``_compute_neighbor_cache_torch`` and the EXPLICIT_GEMM branches of
``_sparse_conv_forward`` / ``_sparse_conv_backward``
(flex_gemm/ops/spconv/sparse_conv3d.py:99-131, 228-281, 293-305, 364-396).
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


def load_reference(ref_root):
    pkg = os.path.join(ref_root, "flex_gemm")
    for name, path in (("flex_gemm", pkg), ("flex_gemm.kernels", os.path.join(pkg, "kernels")),
                       ("flex_gemm.ops", os.path.join(pkg, "ops"))):
        m = types.ModuleType(name)
        m.__path__ = [path]
        sys.modules[name] = m
    sys.modules["flex_gemm"].kernels = sys.modules["flex_gemm.kernels"]
    sys.modules["flex_gemm"].ops = sys.modules["flex_gemm.ops"]
    importlib.import_module("flex_gemm.ops.utils")
    sys.modules["flex_gemm.ops"].utils = sys.modules["flex_gemm.ops.utils"]
    spconv = importlib.import_module("flex_gemm.ops.spconv")
    spconv.set_algorithm(spconv.Algorithm.EXPLICIT_GEMM)
    return spconv


def u32(t):
    return t.view(torch.int32).numpy().view(np.uint32)


def main():
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("FLEXGEMM_REFERENCE")
    if not ref_root:
        raise SystemExit("usage: %s <path to the FlexGEMM source tree>  (or set FLEXGEMM_REFERENCE)" % os.path.basename(__file__))
    spconv = load_reference(ref_root)
    fn = spconv.SparseConv3dFunction
    rng = np.random.default_rng(11)
    geoms = {  # name: (ksize, stride, padding, dilation) -- the three of tests/spconv/out_coords.py:38-40 and two more
        "k3s1p1": ((3, 3, 3), (1, 1, 1), (1, 1, 1), (1, 1, 1)),
        "k3s1p2d2": ((3, 3, 3), (1, 1, 1), (2, 2, 2), (2, 2, 2)),
        "k2s2p0": ((2, 2, 2), (2, 2, 2), (0, 0, 0), (1, 1, 1)),
        "k3s2p1": ((3, 3, 3), (2, 2, 2), (1, 1, 1), (1, 1, 1)),
        "k321s212p101": ((3, 2, 1), (2, 1, 2), (1, 0, 1), (1, 2, 1)),
    }
    inputs = {
        "shell8": (orc.reference_sphere_coords(8), (1, 0, 8, 8, 8)),
        "shell8b2": (orc.shell_coords(8, batch=2), (2, 0, 8, 8, 8)),
    }
    dims = (6, 9, 7)
    pts = np.unique(np.stack([rng.integers(0, 3, 60), rng.integers(0, dims[0], 60), rng.integers(0, dims[1], 60),
                              rng.integers(0, dims[2], 60)], axis=1), axis=0).astype(np.int32)
    inputs["random_b3"] = (pts[rng.permutation(len(pts))], (3, 0) + dims)  # unsorted rows
    inputs["single"] = (np.array([[0, 1, 1, 1]], dtype=np.int32), (1, 0, 3, 3, 3))
    out = {}
    for iname, (coords, shape) in inputs.items():
        for gname, (k, s, p, d) in geoms.items():
            tag = f"{iname}.{gname}"
            c = torch.from_numpy(np.ascontiguousarray(coords))
            oc = fn._get_output_coords_torch(c, torch.Size(shape), k, s, p, d).contiguous()
            out[tag + ".coords"] = coords
            out[tag + ".shape"] = np.array(shape, dtype=np.int64)
            out[tag + ".geom"] = np.array(k + s + p + d, dtype=np.int64)
            out[tag + ".out_coords"] = oc.numpy().astype(np.int32)
            if oc.shape[0] == 0:
                continue  # the reference's map builder does not accept an empty output set
            cache = fn._compute_neighbor_cache_torch(c, oc, torch.Size(shape), k, s, p, d, True)
            out[tag + ".nbr"] = u32(cache["neighbor_map"])
            out[tag + ".nbr_bwd"] = u32(cache["neighbor_map_bwd"])
            if iname in ("shell8", "random_b3") and oc.shape[0] > 0:
                # explicit forward / backward in fp32, Ci = 8, Co = 16
                g = torch.Generator().manual_seed(len(tag))
                V = k[0] * k[1] * k[2]
                feats = torch.randn(coords.shape[0], 8, generator=g).requires_grad_(True)
                weight = (torch.randn(16, k[0], k[1], k[2], 8, generator=g) / (V * 8) ** 0.5).requires_grad_(True)
                bias = torch.randn(16, generator=g).requires_grad_(True)
                gout = torch.randn(oc.shape[0], 16, generator=g)
                y = fn._sparse_conv_forward(feats, cache, weight, bias)
                gi, gw, gb = fn._sparse_conv_backward(gout, feats, cache, weight, bias)
                out[tag + ".feats"] = feats.detach().numpy()
                out[tag + ".weight"] = weight.detach().numpy()
                out[tag + ".bias"] = bias.detach().numpy()
                out[tag + ".gout"] = gout.numpy()
                out[tag + ".out"] = y.detach().numpy()
                out[tag + ".gin"] = gi.detach().numpy()
                out[tag + ".gw"] = gw.detach().numpy()
                out[tag + ".gb"] = gb.detach().numpy()
    np.savez_compressed(os.path.join(HERE, "sparse_conv.npz"), **out)
    print("wrote sparse_conv.npz:", len(out), "arrays;", sum(1 for k in out if k.endswith(".nbr")), "cases")


if __name__ == "__main__":
    main()
