"""Submanifold sparse convolution -- same names as ``flex_gemm.ops.spconv``
(flex_gemm/ops/spconv/__init__.py:1-41), restricted to the submanifold path."""


class Algorithm:
    """Algorithm choices for sparse convolution.  Every implicit-GEMM value
    runs the masked tcgen05 kernels (they compute the same result); only
    EXPLICIT_GEMM is a different code path (gather + library GEMM, kept as a
    cross-check)."""
    EXPLICIT_GEMM = "explicit_gemm"
    IMPLICIT_GEMM = "implicit_gemm"
    IMPLICIT_GEMM_SPLITK = "implicit_gemm_splitk"
    MASKED_IMPLICIT_GEMM = "masked_implicit_gemm"
    MASKED_IMPLICIT_GEMM_SPLITK = "masked_implicit_gemm_splitk"


_ALL_ALGORITHMS = (Algorithm.EXPLICIT_GEMM, Algorithm.IMPLICIT_GEMM, Algorithm.IMPLICIT_GEMM_SPLITK,
                   Algorithm.MASKED_IMPLICIT_GEMM, Algorithm.MASKED_IMPLICIT_GEMM_SPLITK)

ALGORITHM = Algorithm.MASKED_IMPLICIT_GEMM_SPLITK  # default algorithm
HASHMAP_RATIO = 2.0                                # hash slots per input voxel


def set_algorithm(algorithm: str):
    global ALGORITHM
    if algorithm not in _ALL_ALGORITHMS:
        raise ValueError(f"Unsupported algorithm {algorithm}")
    ALGORITHM = algorithm


def set_hashmap_ratio(ratio: float):
    global HASHMAP_RATIO
    if not ratio >= 1.0:
        raise ValueError("hashmap ratio must be >= 1 (the table needs a slot per voxel)")
    HASHMAP_RATIO = ratio


from .submanifold_conv3d import SubMConv3dFunction, SubMConv3dNeighborCache, sparse_submanifold_conv3d  # noqa: E402,F401
