"""CPU-side checks: the library loads, exports what the header declares, and
rejects bad arguments before launching anything."""
import os
import re

import pytest
import torch

from flexgemm_b200 import _build, _cabi
from flexgemm_b200.ops import spconv
from flexgemm_b200.ops.spconv import SubMConv3dFunction

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    _build.build()
    return _cabi.lib()


def test_header_and_binding_agree(lib):
    header = open(os.path.join(ROOT, "include", "flexgemm_b200.h")).read()
    declared = set(re.findall(r"\b(fgb_[a-z0-9_]+)\s*\(", header))
    assert declared == set(_cabi.EXPORTS)
    for name in declared:
        assert hasattr(lib, name), name


def test_version_and_errors(lib):
    assert b"sm_100a" in lib.fgb_version()
    assert _cabi.error_string(0) == "ok"
    assert "null" in _cabi.error_string(-1)
    with pytest.raises(ValueError):
        _cabi.check(-2, "x")
    with pytest.raises(RuntimeError):
        _cabi.check(1001, "x")


def test_per_device_launch_caches(lib):
    """SM count and shared-memory limits are remembered per device, not per process."""
    assert lib.fgb_selftest_device_tables() == 0


def test_size_queries(lib):
    assert lib.fgb_hash_table_bytes(1000, 32) == 8000
    assert lib.fgb_hash_table_bytes(1000, 64) == 12000
    assert lib.fgb_hash_table_bytes(1000, 16) < 0
    assert lib.fgb_hash_table_bytes(-1, 32) < 0
    assert lib.fgb_map_num_blocks(0) == 0
    assert lib.fgb_map_num_blocks(257) == 2
    assert lib.fgb_conv_tile_rows() == 128
    n = 100000   # enough row blocks for every SM: no split-K slabs in the fprop / dgrad workspaces
    assert lib.fgb_conv_workspace_bytes(0, n, 64, 64, 27, _cabi.F16, 1) == 256
    assert lib.fgb_conv_workspace_bytes(0, n, 64, 64, 27, _cabi.F32_IEEE, 1) == 256 + n * 3 * 64 * 4 + 64 * 64 * 27 * 3 * 4
    assert lib.fgb_conv_workspace_bytes(1, n, 64, 32, 27, _cabi.F16, 1) == 256 + 64 * 32 * 27 * 2
    # a launch with fewer work items than SMs is split over the offsets: room for the fp32 slabs [splits, n, Co]
    small = lib.fgb_conv_workspace_bytes(0, 1000, 64, 64, 27, _cabi.F16, 1) - 256
    assert small > 0 and small % (1000 * 64 * 4) == 0 and 2 <= small // (1000 * 64 * 4) <= 27
    assert lib.fgb_conv_workspace_bytes(2, 1000, 64, 32, 27, _cabi.F16, 4) == 64 * 32 * 27 * 4 * 5
    assert lib.fgb_conv_workspace_bytes(2, 1000, 64, 32, 27, 9, 4) < 0
    assert lib.fgb_bias_grad_workspace_bytes(256) > 0


def test_argument_validation_without_launch(lib):
    # all of these return before touching the device
    assert lib.fgb_subm_build_neighbor_map(0, 10, 1, 4, 4, 4, 2, 3, 3, 1, 1, 1, 0, 20, 32, 0, 0, 0, 0, 0, 0, 0) == -2  # even kernel
    assert lib.fgb_subm_build_neighbor_map(0, 10, 1, 4, 4, 4, 3, 3, 5, 1, 1, 1, 0, 20, 32, 0, 0, 0, 0, 0, 0, 0) == -2  # V > 32
    assert lib.fgb_subm_build_neighbor_map(0, 10, 1, 4, 4, 4, 3, 3, 3, 1, 1, 1, 0, 5, 32, 0, 0, 0, 0, 0, 0, 0) == -2   # slots < n
    assert lib.fgb_subm_build_neighbor_map(0, 10, 1, 4, 4, 4, 3, 3, 3, 1, 1, 1, 0, 20, 48, 0, 0, 0, 0, 0, 0, 0) == -3  # key width
    assert lib.fgb_subm_build_neighbor_map(0, 10, 1, 4, 4, 4, 3, 3, 3, 1, 1, 1, 0, 20, 32, 0, 0, 0, 0, 0, 0, 0) == -1  # null seg
    assert lib.fgb_pp_tile_masks(0, 0, 10, 100, 0, 0) == -2   # not a power of two
    assert lib.fgb_subm_conv_fprop(0, 0, 0, 0, 0, 0, 0, 0, 10, 64, 64, 27, _cabi.F16, 0, 0, 0, 0) == -1
    assert lib.fgb_subm_conv_fprop(16, 16, 0, 16, 16, 16, 0, 16, 100000, 60, 64, 27, _cabi.F16, 256, 256, 0, 0) == -4  # Ci % 8
    assert lib.fgb_subm_conv_fprop(16, 16, 0, 16, 16, 16, 0, 16, 100000, 64, 64, 27, 7, 256, 256, 0, 0) == -3
    assert lib.fgb_subm_conv_fprop(16, 16, 0, 16, 16, 16, 0, 16, 10, 64, 64, 27, _cabi.F16, 256, 256, 0, 0) == -5  # small launch: no room for the split-K slabs
    assert lib.fgb_subm_conv_wgrad(16, 16, 16, 16, 16, 0, 16, 0, 10, 100, 64, 64, 27, _cabi.F16, 2, 256, 10, 0, 0) == -5  # workspace
    assert lib.fgb_wgrad_set_row_bands(65) == -2 and lib.fgb_wgrad_set_row_bands(0) == 0


def test_sparse_conv_entry_points_validate_without_launch(lib):
    import ctypes
    wo, ho, do = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    g = (3, 3, 3, 2, 2, 2, 1, 1, 1, 1, 1, 1)
    assert lib.fgb_sparse_out_grid(16, 17, 9, *g, ctypes.byref(wo), ctypes.byref(ho), ctypes.byref(do)) == 0
    assert (wo.value, ho.value, do.value) == (8, 9, 5)   # (n + 2p - d(k-1) - 1) // s + 1
    assert lib.fgb_sparse_out_grid(16, 17, 9, 3, 3, 3, 0, 2, 2, 1, 1, 1, 1, 1, 1, ctypes.byref(wo), ctypes.byref(ho), ctypes.byref(do)) == -2
    assert lib.fgb_sparse_out_coords_collect(0, 10, 8, 8, 8, *g, 0, 100, 48, 0, 16, 0, 0) == -3     # key width
    assert lib.fgb_sparse_out_coords_collect(0, 10, 8, 8, 8, 3, 3, 4, 2, 2, 2, 1, 1, 1, 1, 1, 1, 0, 100, 32, 0, 16, 0, 0) == -2  # V > 32
    assert lib.fgb_sparse_out_coords_collect(0, 10, 8, 8, 8, *g, 0, 100, 32, 0, 0, 0, 0) == -1      # null count
    assert lib.fgb_sparse_out_coords_workspace_bytes(0, 32, 0) == 0
    assert lib.fgb_sparse_out_coords_workspace_bytes(10, 32, 3) == -2
    assert lib.fgb_sparse_out_coords_finalize(16, 5, 32, 1, 0, 1, 8, 8, 8, *g, 256, 1 << 20, 16, 0) == -2   # coord_bits for Morton
    assert lib.fgb_sparse_build_neighbor_map(16, 10, 16, 5, 8, 8, 8, *g, 16, 5, 32, 16, 0, 16, 16, 16, 16, 0, 0) == -2   # slots < n_in
    assert lib.fgb_sparse_build_neighbor_map(16, 10, 16, 5, 8, 8, 8, *g, 16, 20, 32, 16, 0, 16, 16, 16, 0, 0, 0) == -1   # null seg
    assert lib.fgb_pp_gray_code(0, 10, 40, 0, 0, 0) == -2
    no, ni = 100000, 50000   # enough rows on both sides that neither fprop nor dgrad is split
    assert lib.fgb_sparse_conv_workspace_bytes(0, no, ni, 64, 64, 27, _cabi.F32_IEEE, 1) == 256 + ni * 3 * 64 * 4 + 64 * 64 * 27 * 3 * 4
    assert lib.fgb_sparse_conv_workspace_bytes(1, no, ni, 64, 32, 27, _cabi.F32_IEEE, 1) == \
        256 + 64 * 32 * 27 * 4 + 64 * 32 * 27 * 3 * 4 + no * 3 * 32 * 4
    assert lib.fgb_sparse_conv_fprop(16, 16, 0, 16, 16, 16, 0, 16, no, ni, 60, 64, 27, _cabi.F16, 256, 256, 0, 0) == -4  # Ci % 8
    assert lib.fgb_sparse_conv_wgrad(16, 16, 16, 16, 16, 0, 16, 0, 10, 20, 500, 64, 64, 27, _cabi.F16, 2, 256, 10, 0, 0) == -2  # pairs > n_out*V


def test_fused_fprop_validates_without_launch(lib):
    args = lambda act, n=10, ci=64, res=16, pre=16: (16, 16, 0, res, 16, 16, 16, 0, 16, pre, n, ci, 64, 27, _cabi.F16, act, 256, 256, 0, 0)
    assert lib.fgb_subm_conv_fprop_fused(*args(2)) == -2            # unknown activation
    assert lib.fgb_subm_conv_fprop_fused(*args(1, ci=60)) == -4     # Ci % 8
    assert lib.fgb_subm_conv_fprop_fused(*args(1, res=8)) == -4     # residual not 16-byte aligned
    assert lib.fgb_subm_conv_fprop_fused(*args(1, n=0)) == 0        # nothing to do
    assert hasattr(spconv, "sparse_submanifold_conv3d_fused") and hasattr(spconv, "SubMConv3dFusedFunction")


def test_conv_cta_limit_is_a_plain_host_setting(lib):
    assert lib.fgb_conv_set_cta_limit(100) == 0
    assert lib.fgb_conv_set_cta_limit(0) == 100
    assert lib.fgb_conv_set_cta_limit(-1) == -2
    assert lib.fgb_conv_set_cta_limit(0) == 0


def test_python_surface_matches_reference_names():
    for name in ("Algorithm", "ALGORITHM", "HASHMAP_RATIO", "set_algorithm", "set_hashmap_ratio", "SubMConv3dFunction",
                 "SubMConv3dNeighborCache", "sparse_submanifold_conv3d", "SparseConv3dFunction", "SparseConv3dNeighborCache",
                 "sparse_conv3d", "SerializationMode", "SparseConv3dOutCoordAlgorithm", "OUT_COORD_ALGO", "OUT_COORD_HASHMAP_RATIO",
                 "SERIALIZATION_MODE"):
        assert hasattr(spconv, name), name
    for name in ("_compute_neighbor_cache", "_compute_neighbor_cache_torch", "_sparse_submanifold_conv_forward",
                 "_sparse_submanifold_conv_backward"):
        assert hasattr(SubMConv3dFunction, name), name
    assert spconv.ALGORITHM == spconv.Algorithm.MASKED_IMPLICIT_GEMM_SPLITK
    with pytest.raises(ValueError):
        spconv.set_algorithm("winograd")
    with pytest.raises(ValueError):
        spconv.set_hashmap_ratio(0.5)


def test_cpu_tensors_are_rejected_not_emulated():
    coords = torch.zeros((4, 4), dtype=torch.int32)
    with pytest.raises(NotImplementedError):
        SubMConv3dFunction._compute_neighbor_cache(coords, torch.Size((1, 8, 4, 4, 4)), (3, 3, 3), (1, 1, 1), True)
    with pytest.raises(AssertionError):
        SubMConv3dFunction._compute_neighbor_cache(coords.long(), torch.Size((1, 8, 4, 4, 4)), (3, 3, 3), (1, 1, 1), True)


def test_missing_library_fails_loudly(monkeypatch):
    monkeypatch.setattr(_cabi, "_lib", None)
    monkeypatch.setenv("FLEXGEMM_B200_LIB", "/nonexistent/libflexgemm_b200.so")
    with pytest.raises(RuntimeError, match="no fallback"):
        _cabi.lib()


def test_explicit_algorithm_on_cpu_matches_golden():
    """The library-GEMM cross-check path (Algorithm.EXPLICIT_GEMM) against the
    reference-generated fixture."""
    import numpy as np
    gold = np.load(os.path.join(ROOT, "tests", "golden", "conv_explicit.npz"))
    name = "r8_c16_c24_f32"
    t = {k: torch.from_numpy(gold[f"{name}/{k}"]) for k in
         ("coords", "feats", "weight", "bias", "out", "grad_out", "grad_feats", "grad_weight", "grad_bias")}
    shape = torch.Size(gold[name + "/shape"].tolist())
    old = spconv.ALGORITHM
    spconv.set_algorithm(spconv.Algorithm.EXPLICIT_GEMM)
    try:
        cache = SubMConv3dFunction._compute_neighbor_cache_torch(t["coords"], shape, (3, 3, 3), (1, 1, 1))
        f = t["feats"].clone().requires_grad_(True)
        w = t["weight"].clone().requires_grad_(True)
        b = t["bias"].clone().requires_grad_(True)
        out, _ = spconv.sparse_submanifold_conv3d(f, t["coords"], shape, w, b, cache)
        out.backward(t["grad_out"])
    finally:
        spconv.set_algorithm(old)
    assert torch.allclose(out, t["out"], atol=1e-5)
    assert torch.allclose(f.grad, t["grad_feats"], atol=1e-5)
    assert torch.allclose(w.grad, t["grad_weight"], atol=1e-4)
    assert torch.allclose(b.grad, t["grad_bias"], atol=1e-4)


def test_reference_module_paths_and_call_shapes():
    """Names the reference's own scripts reach for: the TF32 switch under its Triton module path
    (tests/submconv/inf_ablation.py:20 there) and init_hashmap's (keys, values) result (ops/utils.py:4-19)."""
    from flexgemm_b200 import kernels
    from flexgemm_b200.kernels import config
    from flexgemm_b200.kernels.triton.spconv import config as ref_path
    from flexgemm_b200.ops import utils
    assert ref_path.allow_tf32 is config.allow_tf32
    try:
        ref_path.allow_tf32 = False
        assert config.allow_tf32 is False and kernels.triton.spconv.config.allow_tf32 is False
    finally:
        config.allow_tf32 = True
    assert ref_path.allow_tf32 is True
    keys, vals = utils.init_hashmap((1, 8, 64, 64, 64), 100, "cpu")
    assert keys.dtype == torch.uint32 and vals.dtype == torch.uint32 and keys.shape == vals.shape == (100,)
    assert int(keys.view(torch.int32)[0]) == -1
    only = utils.init_hashmap((8, 8, 1024, 1024, 1024), 10, "cpu", with_values=False)
    assert only.dtype == torch.uint64 and only.shape == (10,)
