"""Host-side check of how the wgrad kernel splits the pair lists among its CTAs
(row bands shared by all offsets): every pair is read by exactly one CTA of its
offset, a CTA never reads past the end of a band, bands are cut at the same
output rows for every offset, and the CTAs of an offset carry equal loads
(with a single band: equal units and a shorter last one).

The split is replayed on the host by ``fgb_wgrad_plan_host`` from the same
helper functions the kernel uses; no GPU is involved."""
import ctypes

import numpy as np
import pytest

from flexgemm_b200 import _build, _cabi
from oracle import submconv_oracle as orc


@pytest.fixture(scope="module")
def lib():
    _build.build()
    return _cabi.lib()


def block_offsets_of(nbr: np.ndarray) -> np.ndarray:
    """[V, nblk] exclusive prefix over 256-row blocks of the valid pairs per offset (what the map build emits)."""
    n, V = nbr.shape
    nblk = (n + 255) // 256
    valid = nbr != orc.INVALID
    counts = np.zeros((V, nblk), np.uint32)
    for k in range(nblk):
        counts[:, k] = valid[k * 256:(k + 1) * 256].sum(0)
    return np.ascontiguousarray(np.concatenate([np.zeros((V, 1), np.uint32), np.cumsum(counts, 1)[:, :-1].astype(np.uint32)], axis=1))


def plan(lib, seg, boff, n, ci, co, dtype, splitk, forced_bands=0):
    V = seg.shape[0] - 1
    prev = lib.fgb_wgrad_set_row_bands(forced_bands)
    try:
        cap = 4096 * 64 * 3
        out = np.zeros(cap, np.uint32)
        bands, kb = ctypes.c_int(), ctypes.c_int()
        units = lib.fgb_wgrad_plan_host(seg.ctypes.data, boff.ctypes.data if boff is not None else 0, n, n, ci, co, V, dtype, splitk,
                                        out.ctypes.data, cap, ctypes.byref(bands), ctypes.byref(kb))
    finally:
        lib.fgb_wgrad_set_row_bands(prev)
    assert units > 0, units
    return out[:units * bands.value * 3].reshape(units, bands.value, 3), bands.value, kb.value


@pytest.mark.parametrize("res,c,forced", [(32, 64, 0), (32, 64, 7), (64, 256, 0), (64, 256, 16), (64, 512, 64), (24, 32, 3)])
def test_every_pair_is_read_once_and_loads_are_even(lib, res, c, forced):
    coords = orc.shell_coords(res)
    shape = (1, c, res, res, res)
    nbr = orc.neighbor_map(coords, shape)
    vs_i, vs_o, seg = orc.valid_signal(nbr)
    seg = np.ascontiguousarray(seg.astype(np.uint32))
    n, V = nbr.shape
    boff = block_offsets_of(nbr)
    splitk = lib.fgb_wgrad_default_splitk(int(seg[-1]), c, c, V, _cabi.F16)
    p, bands, kb = plan(lib, seg, boff, n, c, c, _cabi.F16, splitk, forced)
    if forced:
        assert bands <= forced
    seen = np.zeros(int(seg[-1]), np.int32)
    # units are offset-major: walk them and attribute each to its offset through the pair positions it reads
    u = 0
    for v in range(V):
        loads = []
        while u < p.shape[0] and (p[u, :, 2] <= seg[v + 1]).all() and (p[u, :, 2] >= seg[v]).all() and p[u, -1, 2] == seg[v + 1]:
            blocks = 0
            for b in range(bands):
                first, cnt, end = (int(x) for x in p[u, b])
                last = min(first + cnt * kb, end)
                if cnt:
                    assert seg[v] <= first < end <= seg[v + 1]
                    assert first + (cnt - 1) * kb < end           # no k-block starts past the band's end
                    seen[first:last] += 1
                    # the band's rows: all pairs of this piece have output rows inside the band's row range
                    rows = vs_o[first:last]
                    lo_row = b * (-(-((n + 255) // 256) // bands)) * 256
                    assert rows.min() >= lo_row
                blocks += cnt
            loads.append(blocks)
            u += 1
            if u < p.shape[0] and p[u, 0, 0] == seg[v + 1] and seg[v + 1] < seg[-1]:
                break
        assert loads, v
        if bands == 1:   # one band: full units and a shorter last one
            assert len(set(loads[:-1])) <= 1 and loads[-1] <= loads[0], (v, loads)
        else:            # several bands: the remainders are dealt round-robin, totals differ by at most one block
            assert max(loads) - min(loads) <= 1, (v, loads)
    assert u == p.shape[0]
    assert (seen == 1).all()


def test_without_block_offsets_there_is_one_band(lib):
    coords = orc.shell_coords(32)
    nbr = orc.neighbor_map(coords, (1, 64, 32, 32, 32))
    _, _, seg = orc.valid_signal(nbr)
    seg = np.ascontiguousarray(seg.astype(np.uint32))
    p, bands, kb = plan(lib, seg, None, nbr.shape[0], 64, 64, _cabi.F16, 4)
    assert bands == 1
    seen = np.zeros(int(seg[-1]), np.int32)
    for first, cnt, end in p[:, 0]:
        seen[int(first):min(int(first) + int(cnt) * kb, int(end))] += 1
    assert (seen == 1).all()
