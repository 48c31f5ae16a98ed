"""Builds the reference's own CUDA extension from its sources, where they lie,
into ``oracle/_ref/flex_gemm_ref_cuda.so`` (test infrastructure: a checker and a
baseline, never part of the product; nothing is copied, only the object code
lands in this repository's ignored ``oracle/_ref``).

    python oracle/build_reference_ext.py <path to the FlexGEMM source tree>

The extension is a plain nvcc + pybind11 module (its setup.py lists seven source
files: kernels/cuda/{hash/hash.cu, serialize/api.cu, grid_sample/grid_sample.cu,
spconv/subm_neighbor_map.cu, spconv/sparse_neighbor_map.cu,
spconv/migemm_neighmap_pp.cu, ext.cpp}); this recipe compiles those files with
the flags of that setup.py (-O3 -std=c++17 --use_fast_math) for sm_100 and links
them against the torch libraries of the running interpreter.  The module is
then loaded by path under the name ``flex_gemm_ref_cuda`` (see
``load_reference_ext``): it exposes the reference's table, neighbour-map and
post-processing functions, which produce the fixtures of
tests/golden/postprocess.npz and time the reference's map build on the GPU.
"""
import importlib.util
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
NAME = "flex_gemm_ref_cuda"
OUT = os.path.join(OUT_DIR, NAME + ".so")
SOURCES = ["hash/hash.cu", "serialize/api.cu", "grid_sample/grid_sample.cu", "spconv/subm_neighbor_map.cu",
           "spconv/sparse_neighbor_map.cu", "spconv/migemm_neighmap_pp.cu", "ext.cpp"]


def build(ref_root: str, force: bool = False) -> str:
    import torch
    from torch.utils import cpp_extension as ce
    src_dir = os.path.join(ref_root, "flex_gemm", "kernels", "cuda")
    srcs = [os.path.join(src_dir, s) for s in SOURCES]
    for s in srcs:
        if not os.path.exists(s):
            raise FileNotFoundError(s)
    os.makedirs(OUT_DIR, exist_ok=True)
    if not force and os.path.exists(OUT) and os.path.getmtime(OUT) >= max(os.path.getmtime(s) for s in srcs):
        return OUT
    inc = [f"-I{p}" for p in ce.include_paths(device_type="cuda")] + [f"-I{sysconfig.get_paths()['include']}"]
    abi = "1" if torch.compiled_with_cxx11_abi() else "0"
    common = ["-O3", "-std=c++17", f"-D_GLIBCXX_USE_CXX11_ABI={abi}", f"-DTORCH_EXTENSION_NAME={NAME}", "-DTORCH_API_INCLUDE_EXTENSION_H"]
    nvcc = os.environ.get("NVCC", "nvcc")
    objs, procs = [], []
    for s in srcs:
        o = os.path.join(OUT_DIR, "ref_" + os.path.basename(s).replace(".", "_") + ".o")
        objs.append(o)
        cmd = [nvcc, "-gencode", "arch=compute_100,code=sm_100", "--use_fast_math", "-allow-unsupported-compiler", "-Xcompiler", "-fPIC",
               "-x", "cu" if s.endswith(".cu") else "c++", "--expt-relaxed-constexpr", "-w"] + common + inc + ["-c", s, "-o", o]
        procs.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for cmd, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            raise RuntimeError("nvcc failed: %s\n%s" % (" ".join(cmd), out[-4000:]))
    libs = [f"-L{p}" for p in ce.library_paths(device_type="cuda")]
    link = [nvcc, "-shared", "-o", OUT] + objs + libs + ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python"]
    r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError("link failed: %s\n%s" % (" ".join(link), r.stdout[-4000:]))
    for o in objs:
        os.remove(o)
    return OUT


def load_reference_ext():
    """The built module, or None when it is not there (it is only ever built where the reference tree is)."""
    if not os.path.exists(OUT):
        return None
    import torch  # noqa: F401  (the module links against the torch libraries)
    spec = importlib.util.spec_from_file_location(NAME, OUT)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def reference_neighbor_cache(ref, coords, shape, ksize=(3, 3, 3), dilation=(1, 1, 1), ratio=2.0):
    """The reference's own cache construction for the masked algorithm with needs_grad=True
    (flex_gemm/ops/spconv/submanifold_conv3d.py:45-97), through its compiled functions:
    -> (neighbor_map, gray_code, sorted_idx, valid_signal_i, valid_signal_o, valid_signal_seg)."""
    import torch
    N, C, W, H, D = [int(v) for v in shape]
    n = coords.shape[0]
    kdt = torch.uint32 if N * W * H * D < 2 ** 32 else torch.uint64          # flex_gemm/ops/utils.py:4-19
    keys = torch.full((int(ratio * n),), torch.iinfo(kdt).max, dtype=kdt, device=coords.device)
    vals = torch.empty((int(ratio * n),), dtype=torch.uint32, device=coords.device)
    nbr = ref.hashmap_build_submanifold_conv_neighbour_map(keys, vals, coords, W, H, D, *ksize, *dilation)
    return (nbr, *ref.neighbor_map_post_process_for_masked_implicit_gemm_1(nbr))


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("FLEXGEMM_REFERENCE")
    if not root:
        raise SystemExit("usage: build_reference_ext.py <path to the FlexGEMM source tree>  (or set FLEXGEMM_REFERENCE)")
    print(build(root, force="--force" in sys.argv))
