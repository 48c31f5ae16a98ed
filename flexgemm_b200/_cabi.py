"""ctypes binding of ``libflexgemm_b200.so`` (declarations: include/flexgemm_b200.h).

Only plain integers and raw device pointers cross this boundary.  There is no
fallback: if the library is missing, loading raises and every op fails.
"""
import ctypes
import os
from ctypes import c_char_p, c_int, c_int64, c_void_p

from . import _build

OK = 0
S_TABLE_FULL = 1
S_WAIT_TIMEOUT = 2
F16, BF16, F32_TF32, F32_IEEE = 0, 1, 2, 3

_P = c_void_p
_PROTOTYPES = {
    "fgb_version": (c_char_p, []),
    "fgb_error_string": (c_char_p, [c_int]),
    "fgb_selftest_device_tables": (c_int, []),
    "fgb_fetch_words_async": (c_int, [_P, _P, c_int64, _P]),
    "fgb_microbench_pipeline": (c_int, [c_int, c_int, c_int, c_int, c_int, _P, c_int64, c_int, _P, c_int64, _P, _P, _P, _P]),
    "fgb_hash_table_bytes": (c_int64, [c_int64, c_int]),
    "fgb_map_num_blocks": (c_int64, [c_int64]),
    "fgb_subm_build_neighbor_map": (c_int, [_P, c_int64, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                            _P, c_int64, c_int, _P, _P, _P, _P, _P, _P, _P]),
    "fgb_pp_sorted_idx_workspace_bytes": (c_int64, [c_int64]),
    "fgb_pp_sorted_idx": (c_int, [_P, c_int64, c_int, _P, _P, c_int64, _P, _P]),
    "fgb_pp_valid_signal": (c_int, [_P, _P, c_int64, c_int, _P, _P, _P, _P, _P, _P]),
    "fgb_pp_tile_masks": (c_int, [_P, _P, c_int64, c_int, _P, _P]),
    "fgb_pp_valid_kernel": (c_int, [_P, c_int64, _P, _P, _P]),
    "fgb_conv_tile_rows": (c_int, []),
    "fgb_conv_block_schedule": (c_int, [_P, c_int64, _P, _P]),
    "fgb_conv_set_cta_limit": (c_int, [c_int]),
    "fgb_conv_set_splitk": (c_int, [c_int]),
    "fgb_conv_set_dgrad_relayout": (c_int, [c_int]),
    "fgb_subm_conv_fprop": (c_int, [_P, _P, _P, _P, _P, _P, _P, _P, c_int64, c_int, c_int, c_int, c_int, _P, c_int64, _P, _P]),
    "fgb_subm_conv_fprop_fused": (c_int, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, c_int64, c_int, c_int, c_int, c_int, c_int, _P, c_int64,
                                          _P, _P]),
    "fgb_subm_conv_dgrad": (c_int, [_P, _P, _P, _P, _P, _P, _P, c_int64, c_int, c_int, c_int, c_int, _P, c_int64, _P, _P]),
    "fgb_conv_workspace_bytes": (c_int64, [c_int, c_int64, c_int, c_int, c_int, c_int, c_int]),
    "fgb_wgrad_default_splitk": (c_int, [c_int64, c_int, c_int, c_int, c_int]),
    "fgb_subm_conv_wgrad": (c_int, [_P, _P, _P, _P, _P, _P, _P, _P, c_int64, c_int64, c_int, c_int, c_int, c_int, c_int, _P, c_int64, _P, _P]),
    "fgb_wgrad_set_row_bands": (c_int, [c_int]),
    "fgb_wgrad_plan_host": (c_int, [_P, _P, c_int64, c_int64, c_int, c_int, c_int, c_int, c_int, _P, c_int64, _P, _P]),
    "fgb_bias_grad_workspace_bytes": (c_int64, [c_int]),
    "fgb_subm_conv_bias_grad": (c_int, [_P, _P, _P, c_int64, c_int, c_int, _P, c_int64, _P]),
    "fgb_cast_from_f32": (c_int, [_P, _P, c_int64, c_int, _P]),
    "fgb_hash_insert_3d_idx_as_val": (c_int, [_P, c_int64, c_int, c_int, c_int, _P, c_int64, c_int, _P, _P]),
    "fgb_hash_lookup_3d": (c_int, [_P, c_int64, c_int, c_int, c_int, _P, c_int64, c_int, _P, _P]),
    "fgb_hashmap_insert": (c_int, [_P, _P, c_int64, c_int, c_int, _P, _P, c_int64, _P, _P]),
    "fgb_hashmap_lookup": (c_int, [_P, _P, c_int64, c_int, c_int, _P, c_int64, _P, _P]),
    "fgb_hashmap_insert_3d": (c_int, [_P, _P, c_int64, c_int, c_int, _P, _P, c_int64, c_int, c_int, c_int, _P, _P]),
    "fgb_hashmap_insert_3d_idx_as_val": (c_int, [_P, _P, c_int64, c_int, c_int, _P, c_int64, c_int, c_int, c_int, _P, _P]),
    "fgb_hashmap_lookup_3d": (c_int, [_P, _P, c_int64, c_int, c_int, _P, c_int64, c_int, c_int, c_int, _P, _P]),
    "fgb_grid_sample_neighbor_map": (c_int, [_P, c_int64, c_int64, c_int, c_int, c_int, _P, c_int64, c_int, c_int, _P, _P, _P]),
    "fgb_indice_weighted_sum_fwd": (c_int, [_P, _P, _P, _P, c_int64, c_int, c_int, c_int, _P]),
    "fgb_indice_weighted_sum_bwd": (c_int, [_P, _P, _P, _P, c_int64, c_int64, c_int, c_int, c_int, _P]),
    "fgb_sparse_out_grid": (c_int, [c_int] * 15 + [_P, _P, _P]),
    "fgb_sparse_out_coords_collect": (c_int, [_P, c_int64] + [c_int] * 15 + [_P, c_int64, c_int, _P, _P, _P, _P]),
    "fgb_sparse_out_coords_workspace_bytes": (c_int64, [c_int64, c_int, c_int]),
    "fgb_sparse_out_coords_finalize": (c_int, [_P, c_int64, c_int, c_int, c_int, c_int] + [c_int] * 15 + [_P, c_int64, _P, _P]),
    "fgb_sparse_build_neighbor_map": (c_int, [_P, c_int64, _P, c_int64] + [c_int] * 15 + [_P, c_int64, c_int, _P, _P, _P, _P, _P, _P, _P, _P]),
    "fgb_pp_gray_code": (c_int, [_P, c_int64, c_int, _P, _P, _P]),
    "fgb_sparse_conv_fprop": (c_int, [_P, _P, _P, _P, _P, _P, _P, _P, c_int64, c_int64, c_int, c_int, c_int, c_int, _P, c_int64, _P, _P]),
    "fgb_sparse_conv_dgrad": (c_int, [_P, _P, _P, _P, _P, _P, _P, c_int64, c_int64, c_int, c_int, c_int, c_int, _P, c_int64, _P, _P]),
    "fgb_sparse_conv_wgrad": (c_int, [_P, _P, _P, _P, _P, _P, _P, _P, c_int64, c_int64, c_int64, c_int, c_int, c_int, c_int, c_int, _P, c_int64, _P, _P]),
    "fgb_sparse_conv_workspace_bytes": (c_int64, [c_int, c_int64, c_int64, c_int, c_int, c_int, c_int, c_int]),
    "fgb_noalloc_max_channels": (c_int, []),
    "fgb_subm_conv_bias_grad_noalloc": (c_int, [_P, _P, _P, c_int64, c_int, c_int, _P]),
}

EXPORTS = tuple(sorted(_PROTOTYPES))
_lib = None


def library_path() -> str:
    return os.environ.get("FLEXGEMM_B200_LIB", _build.LIB_PATH)


def lib():
    """The loaded library; raises if it has not been built."""
    global _lib
    if _lib is None:
        path = library_path()
        if not os.path.exists(path):
            raise RuntimeError(
                f"{path} not found: build it with `python -m flexgemm_b200._build` "
                "(flexgemm_b200 has no fallback implementation)")
        handle = ctypes.CDLL(path)
        for name, (res, args) in _PROTOTYPES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def error_string(code: int) -> str:
    return lib().fgb_error_string(int(code)).decode()


def check(code: int, what: str) -> None:
    """Raise for a non-zero return code of an int-returning entry point."""
    if code != OK:
        exc = ValueError if code < 0 else RuntimeError
        raise exc(f"{what} failed: {error_string(code)} (code {code})")


def check_size(value: int, what: str) -> int:
    """Entry points that return a byte count report errors as negative values."""
    if value < 0:
        raise ValueError(f"{what} failed: {error_string(int(value))} (code {value})")
    return int(value)
