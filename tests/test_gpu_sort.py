"""The library's own radix argsort (``fgb_pp_sorted_idx``) through the C ABI:
bit-exact against numpy's stable argsort for random and clustered codes, every
pass count (key widths 5 ... 32 bits), both tile sizes, ragged lengths, and
signed codes when all 32 bits are in use."""
import numpy as np
import pytest
import torch

from flexgemm_b200 import _cabi

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def argsort_gpu(codes_np, key_bits):
    lib = _cabi.lib()
    n = codes_np.shape[0]
    codes = torch.from_numpy(codes_np).to(DEV)
    out = torch.full((n,), -1, dtype=torch.int64, device=DEV)
    nbytes = _cabi.check_size(lib.fgb_pp_sorted_idx_workspace_bytes(n), "workspace")
    ws = torch.empty((nbytes + 7) // 8, dtype=torch.int64, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    rc = lib.fgb_pp_sorted_idx(codes.data_ptr(), n, key_bits, out.data_ptr(), ws.data_ptr(), ws.numel() * 8, status.data_ptr(),
                               torch.cuda.current_stream(DEV).cuda_stream)
    _cabi.check(rc, "fgb_pp_sorted_idx")
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    return out.cpu().numpy()


@pytest.mark.parametrize("n", [1, 31, 1000, 1025, 163736, (1 << 20) + 4097])
@pytest.mark.parametrize("key_bits", [5, 9, 18, 27, 32])
def test_argsort_matches_numpy_stable(n, key_bits):
    rng = np.random.default_rng(n + key_bits)
    if key_bits == 32:
        codes = rng.integers(-2 ** 31, 2 ** 31, size=n, dtype=np.int64).astype(np.int32)
    else:
        codes = rng.integers(0, 2 ** key_bits, size=n, dtype=np.int64).astype(np.int32)
    got = argsort_gpu(codes, key_bits)
    assert np.array_equal(got, np.argsort(codes, kind="stable"))


@pytest.mark.parametrize("n", [5000, 300000, (1 << 21) + 77])
def test_argsort_of_clustered_codes(n):
    """Few distinct codes in long runs, as neighbouring voxels produce them (every key of a warp in one digit bin)."""
    rng = np.random.default_rng(7)
    distinct = rng.integers(0, 2 ** 27, size=37, dtype=np.int64).astype(np.int32)
    runs = rng.integers(1, 400, size=n // 100 + 1)
    codes = np.repeat(distinct[rng.integers(0, 37, size=runs.size)], runs)[:n]
    assert codes.shape[0] == n
    got = argsort_gpu(np.ascontiguousarray(codes), 27)
    assert np.array_equal(got, np.argsort(codes, kind="stable"))


def test_all_equal_and_already_sorted():
    n = 70000
    assert np.array_equal(argsort_gpu(np.full(n, 12345, np.int32), 27), np.arange(n))
    asc = np.arange(n, dtype=np.int32)
    assert np.array_equal(argsort_gpu(asc, 27), np.arange(n))
    assert np.array_equal(argsort_gpu(asc[::-1].copy(), 27), np.arange(n)[::-1])
