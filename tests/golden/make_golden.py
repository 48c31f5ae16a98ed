"""Generate the golden vectors under tests/golden/ from the reference itself.

Run once, in a container where the FlexGEMM tree is available:

    python tests/golden/make_golden.py /path/to/FlexGEMM

The reference package cannot be imported normally on a machine without a GPU
(it queries the CUDA device at import), so only its pure-torch pieces are
loaded: ``flex_gemm.ops.spconv`` is imported with ``flex_gemm`` and
``flex_gemm.kernels`` registered as empty stand-in modules.  What is executed
is the reference's own ``_compute_neighbor_cache_torch`` and its
EXPLICIT_GEMM forward/backward, unmodified.  One shim is needed on CPU:
``torch.flip`` has no uint32 kernel, so the call is routed through an int32
view (bit-identical).

The outputs are small ``.npz`` files committed next to this script; the tests
never need the reference tree.
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
    # sparse_conv3d imports serialize helpers that need the compiled extension;
    # it is not on the path, so give it an empty stand-in.
    stub = types.ModuleType("flex_gemm.ops.spconv.sparse_conv3d")
    stub.SparseConv3dFunction = None
    stub.sparse_conv3d = None
    sys.modules["flex_gemm.ops.spconv.sparse_conv3d"] = stub
    spconv = importlib.import_module("flex_gemm.ops.spconv")
    spconv.set_algorithm(spconv.Algorithm.EXPLICIT_GEMM)
    return spconv


_flip = torch.flip


def _flip_u32(x, dims):
    if x.dtype == torch.uint32:
        return _flip(x.view(torch.int32), dims).view(torch.uint32)
    return _flip(x, dims)


def ref_map(spconv, coords, shape, ksize, dil):
    fn = spconv.SubMConv3dFunction
    cache = fn._compute_neighbor_cache_torch(torch.from_numpy(coords), torch.Size(shape), ksize, dil)
    return cache, cache["neighbor_map"].view(torch.int32).numpy().view(np.uint32)


def main():
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("FLEXGEMM_REFERENCE")
    if not ref_root:
        raise SystemExit("usage: %s <path to the FlexGEMM source tree>  (or set FLEXGEMM_REFERENCE)" % os.path.basename(__file__))
    spconv = load_reference(ref_root)
    fn = spconv.SubMConv3dFunction
    torch.flip = _flip_u32

    # ---- neighbour maps ---------------------------------------------------
    maps = {}
    rng = np.random.default_rng(7)
    cases = []
    for res in (1, 2, 4, 8, 16):  # the reference's own shell rule, tests/submconv/neighbor_cache.py:54
        cases.append((f"refshell_r{res}", orc.reference_sphere_coords(res), (1, 0, res, res, res), (3, 3, 3), (1, 1, 1)))
    cases.append(("shell_r16_b2", orc.shell_coords(16, batch=2, scales=(1.0, 0.8)), (2, 0, 16, 16, 16), (3, 3, 3), (1, 1, 1)))
    cases.append(("shell_r32", orc.shell_coords(32), (1, 0, 32, 32, 32), (3, 3, 3), (1, 1, 1)))
    cases.append(("shell_r16_dil2", orc.shell_coords(16), (1, 0, 16, 16, 16), (3, 3, 3), (2, 1, 2)))
    # unsorted random occupancy of a non-cubic grid, two samples
    W, H, D = 7, 5, 9
    occ = rng.random((2, W, H, D)) < 0.35
    c = np.argwhere(occ).astype(np.int32)
    c = np.ascontiguousarray(c[rng.permutation(c.shape[0])])
    cases.append(("random_7x5x9_b2", c, (2, 0, W, H, D), (3, 3, 3), (1, 1, 1)))
    cases.append(("random_7x5x9_k313", c, (2, 0, W, H, D), (3, 1, 3), (1, 1, 1)))
    for name, coords, shape, ks, dil in cases:
        _, m = ref_map(spconv, coords, shape, ks, dil)
        maps[name + "/coords"] = coords
        maps[name + "/shape"] = np.asarray(shape, np.int64)
        maps[name + "/ksize"] = np.asarray(ks, np.int64)
        maps[name + "/dilation"] = np.asarray(dil, np.int64)
        maps[name + "/neighbor_map"] = m
    np.savez_compressed(os.path.join(HERE, "neighbor_maps.npz"), **maps)

    # ---- forward / backward through the reference's explicit path ----------
    conv = {}
    for name, res, ci, co, dtype, seed in (("r8_c16_c24_f32", 8, 16, 24, "float32", 11),
                                           ("r16_c32_c32_f32", 16, 32, 32, "float32", 12),
                                           ("r12_c64_c32_f16", 12, 64, 32, "float16", 13)):
        coords, feats, weight, bias, shape = orc.make_problem(res, ci, co, dtype, seed)
        g = torch.Generator().manual_seed(seed + 100)
        cache = fn._compute_neighbor_cache_torch(coords, torch.Size(shape), (3, 3, 3), (1, 1, 1))
        feats_r = feats.clone().requires_grad_(True)
        weight_r = weight.clone().requires_grad_(True)
        bias_r = bias.clone().requires_grad_(True)
        out = fn._sparse_submanifold_conv_forward(feats_r, cache, weight_r, bias_r)
        gout = torch.randn(out.shape, generator=g).to(out.dtype)
        gin, gw, gb = fn._sparse_submanifold_conv_backward(gout, feats_r, cache, weight_r, bias_r)
        for k, v in (("coords", coords), ("feats", feats), ("weight", weight), ("bias", bias),
                     ("out", out.detach()), ("grad_out", gout), ("grad_feats", gin), ("grad_weight", gw),
                     ("grad_bias", gb)):
            conv[f"{name}/{k}"] = v.detach().numpy()
        conv[f"{name}/shape"] = np.asarray(shape, np.int64)
    np.savez_compressed(os.path.join(HERE, "conv_explicit.npz"), **conv)
    print("wrote", sorted(os.listdir(HERE)))


if __name__ == "__main__":
    main()
