"""Sparse convolution -- same names as ``flex_gemm.ops.spconv``
(flex_gemm/ops/spconv/__init__.py:1-41): the submanifold conv and the generic
strided conv."""


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


class SerializationMode:
    """Serialization mode when constructing a key from 3D coordinates (orders the
    generated output coordinates of ``sparse_conv3d``)."""
    BXYZ = 0
    Z_ORDER = 1
    HILBERT = 2


class SparseConv3dOutCoordAlgorithm:
    """Algorithm choices for generating output coordinates (both run the same
    hash-set kernel here; the results are identical by definition)."""
    HASHMAP = 0
    EXPAND_UNIQUE = 1


_ALL_ALGORITHMS = (Algorithm.EXPLICIT_GEMM, Algorithm.IMPLICIT_GEMM, Algorithm.IMPLICIT_GEMM_SPLITK,
                   Algorithm.MASKED_IMPLICIT_GEMM, Algorithm.MASKED_IMPLICIT_GEMM_SPLITK)

ALGORITHM = Algorithm.MASKED_IMPLICIT_GEMM_SPLITK  # default algorithm
HASHMAP_RATIO = 2.0                                # hash slots per input voxel
OUT_COORD_HASHMAP_RATIO = 1.1                      # hash-set slots per potential output coordinate
OUT_COORD_ALGO = SparseConv3dOutCoordAlgorithm.HASHMAP
SERIALIZATION_MODE = SerializationMode.BXYZ


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
from .sparse_conv3d import SparseConv3dFunction, SparseConv3dNeighborCache, sparse_conv3d  # noqa: E402,F401
from .fused_conv3d import SubMConv3dFusedFunction, sparse_submanifold_conv3d_fused  # noqa: E402,F401
