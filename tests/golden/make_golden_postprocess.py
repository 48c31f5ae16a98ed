"""Generates tests/golden/postprocess.npz: outputs of the REFERENCE's own CUDA
functions for the neighbour cache of the masked implicit GEMM, on seeded inputs.

Runs on a machine with a GPU, with the reference's extension built by
``oracle/build_reference_ext.py`` (the reference tree itself is not needed at
run time):

    python tests/golden/make_golden_postprocess.py [output.npz]

For each case it follows the reference's own call sequence
(flex_gemm/ops/spconv/submanifold_conv3d.py:45-107 and :14-17):
``init_hashmap`` -> ``hashmap_build_submanifold_conv_neighbour_map`` ->
``neighbor_map_post_process_for_masked_implicit_gemm_1`` -> ``..._2`` for tile
sizes 128 and 32, and stores coords, shape, stencil, neighbor_map, gray_code,
sorted_idx, valid_signal_{i,o,seg}, valid_kernel_B and valid_kernel_seg_B.
The fixture pins the oracle's restatement of migemm_neighmap_pp.cu
(tests/test_oracle.py) and, through it, the CUDA path.

It also prints how long the reference's own kernels take to build the cache of
the headline shell on this GPU (a number for the record, not a fixture)."""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import submconv_oracle as orc  # noqa: E402  (input generators only)
from oracle.build_reference_ext import load_reference_ext, reference_neighbor_cache as reference_cache  # noqa: E402


def u32(t):
    return t.cpu().view(torch.int32).numpy().view(np.uint32)


def main():
    ref = load_reference_ext()
    if ref is None:
        raise SystemExit("oracle/_ref/flex_gemm_ref_cuda.so not found: build it with oracle/build_reference_ext.py")
    dev = torch.device("cuda:0")
    out_path = sys.argv[1] if len(sys.argv) > 1 else os.path.join(os.path.dirname(os.path.abspath(__file__)), "postprocess.npz")
    rng = np.random.default_rng(11)
    cases = {}
    cases["shell16"] = (orc.shell_coords(16), (1, 8, 16, 16, 16), (3, 3, 3), (1, 1, 1))
    cases["shell32"] = (orc.shell_coords(32), (1, 8, 32, 32, 32), (3, 3, 3), (1, 1, 1))
    cases["refsphere24_b2"] = (orc.reference_sphere_coords(24, batch=2), (2, 8, 24, 24, 24), (3, 3, 3), (1, 1, 1))
    sh = orc.shell_coords(20, batch=2, scales=(1.0, 0.7))
    cases["shell20_b2_shuffled"] = (np.ascontiguousarray(sh[rng.permutation(sh.shape[0])]), (2, 8, 20, 20, 20), (3, 3, 3), (1, 1, 1))
    cases["shell24_dil2"] = (orc.shell_coords(24), (1, 8, 24, 24, 24), (3, 3, 3), (2, 1, 2))
    cases["shell16_k313"] = (orc.shell_coords(16), (1, 8, 16, 16, 16), (3, 1, 3), (1, 1, 1))
    dense = np.stack(np.meshgrid(np.arange(6), np.arange(5), np.arange(7), indexing="ij"), -1).reshape(-1, 3)
    cases["dense_6x5x7"] = (np.concatenate([np.zeros((dense.shape[0], 1), int), dense], 1).astype(np.int32), (1, 8, 6, 5, 7), (3, 3, 3), (1, 1, 1))
    cases["single_voxel"] = (np.array([[0, 3, 3, 3]], np.int32), (1, 8, 8, 8, 8), (3, 3, 3), (1, 1, 1))
    store = {}
    for name, (coords_np, shape, ks, dil) in cases.items():
        coords = torch.from_numpy(np.ascontiguousarray(coords_np.astype(np.int32))).to(dev)
        nbr, gray, sidx, vs_i, vs_o, seg = reference_cache(ref, coords, shape, ks, dil)
        store[f"{name}/coords"] = coords_np.astype(np.int32)
        store[f"{name}/shape"] = np.array(shape, np.int64)
        store[f"{name}/ksize"] = np.array(ks, np.int64)
        store[f"{name}/dilation"] = np.array(dil, np.int64)
        store[f"{name}/neighbor_map"] = u32(nbr)
        store[f"{name}/gray_code"] = gray.cpu().numpy()
        store[f"{name}/sorted_idx"] = sidx.cpu().numpy()
        store[f"{name}/valid_signal_i"] = u32(vs_i)
        store[f"{name}/valid_signal_o"] = u32(vs_o)
        store[f"{name}/valid_signal_seg"] = u32(seg)
        for block in (128, 32):
            vk, vks = ref.neighbor_map_post_process_for_masked_implicit_gemm_2(gray, sidx, block)
            store[f"{name}/valid_kernel_{block}"] = vk.cpu().numpy()
            store[f"{name}/valid_kernel_seg_{block}"] = vks.cpu().numpy()
        print(name, coords_np.shape[0], "voxels,", int(u32(seg)[-1]), "pairs")
    np.savez_compressed(out_path, **store)
    print("wrote", out_path)

    # for the record: the reference's own cache build on this GPU (its hash table, neighbour map and post-processing)
    for label, coords_np, shape in (("RES=256 shell", orc.shell_coords(256), (1, 256, 256, 256, 256)),):
        coords = torch.from_numpy(coords_np).to(dev)
        for _ in range(3):
            reference_cache(ref, coords, shape, (3, 3, 3), (1, 1, 1))
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(20):
            reference_cache(ref, coords, shape, (3, 3, 3), (1, 1, 1))
        b.record()
        torch.cuda.synchronize()
        print(f"reference cache build, {label}: {a.elapsed_time(b) / 20:.4f} ms")


if __name__ == "__main__":
    main()
