"""Generate tests/golden/serialize_keys.npz: Morton and Hilbert keys computed
by the reference's own headers (flex_gemm/kernels/cuda/serialize/z_order.h,
hilbert.h), compiled as host code through ``oracle/ref_serialize.cu``.

    python tests/golden/make_golden_serialize.py /path/to/FlexGEMM
"""
import os
import subprocess
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.abspath(os.path.join(HERE, "..", ".."))


def main():
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("FLEXGEMM_REFERENCE")
    if not ref_root:
        raise SystemExit("usage: %s <path to the FlexGEMM source tree>  (or set FLEXGEMM_REFERENCE)" % os.path.basename(__file__))
    exe = os.path.join(ROOT, "oracle", "_ref", "ref_serialize")
    os.makedirs(os.path.dirname(exe), exist_ok=True)
    subprocess.run(["nvcc", "-O1", "-I" + os.path.join(ref_root, "flex_gemm", "kernels", "cuda"), "-o", exe,
                    os.path.join(ROOT, "oracle", "ref_serialize.cu")], check=True, stderr=subprocess.DEVNULL)
    rng = np.random.default_rng(3)
    out = {}
    for bits in (1, 2, 3, 5, 8, 10, 12, 21):
        n = 8 if bits == 1 else 200
        pts = rng.integers(0, 1 << bits, size=(n, 3), dtype=np.int64)
        if bits <= 2:  # every point of the cube
            g = np.arange(1 << bits)
            pts = np.stack(np.meshgrid(g, g, g, indexing="ij"), axis=-1).reshape(-1, 3)
        b = rng.integers(0, 4, size=(pts.shape[0], 1), dtype=np.int64)
        coords = np.concatenate([b, pts], axis=1)
        text = f"{bits} {coords.shape[0]}\n" + "\n".join(" ".join(str(int(v)) for v in row) for row in coords) + "\n"
        res = subprocess.run([exe], input=text, capture_output=True, text=True, check=True)
        vals = np.array([[int(t) for t in line.split()] for line in res.stdout.strip().splitlines()], dtype=np.uint64)
        fits32 = bits * 3 + 2 < 32
        if fits32:  # the 32-bit and the 64-bit instantiation agree wherever the former applies
            assert np.array_equal(vals[:, 0], vals[:, 2]) and np.array_equal(vals[:, 1], vals[:, 3])
        out[f"bits{bits}.coords"] = coords.astype(np.int32)
        out[f"bits{bits}.morton"] = vals[:, 0]
        out[f"bits{bits}.hilbert"] = vals[:, 1]
    np.savez_compressed(os.path.join(HERE, "serialize_keys.npz"), **out)
    print("wrote serialize_keys.npz:", len(out), "arrays")


if __name__ == "__main__":
    main()
