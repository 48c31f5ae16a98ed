"""Sparse grid sample -- same names as ``flex_gemm.ops.grid_sample``
(flex_gemm/ops/grid_sample/__init__.py:1-10)."""

HASHMAP_RATIO = 2.0         # hash slots per input voxel


def set_hashmap_ratio(ratio: float):
    global HASHMAP_RATIO
    if not ratio >= 1.0:
        raise ValueError("hashmap ratio must be >= 1 (the table needs a slot per voxel)")
    HASHMAP_RATIO = ratio


from .grid_sample_torch import grid_sample_3d_torch  # noqa: E402,F401
from .grid_sample import GridSample3dFunction, grid_sample_3d  # noqa: E402,F401
