"""Seeded synthetic workloads of the benchmark family (spherical voxel shells).

The reference measures on synthetic spherical shells generated on the fly
(tests/utils.py:5-25 in its tree), not on a dataset; these generators produce
the shells of the same family that the benchmark configurations name."""
import math
from typing import Optional, Sequence, Tuple

import numpy as np
import torch


def shell_coords(res: int, batch: int = 1, scales: Optional[Sequence[float]] = None) -> np.ndarray:
    """int32 [N,4] rows (b,x,y,z), lexicographic: every voxel of [0,res)^3 whose
    centre is at distance d from the grid centre with r-1 < d <= r,
    r = 0.45 * res * scale (float32 distance arithmetic)."""
    if scales is None:
        scales = [1.0] * batch
    ax = (np.arange(res, dtype=np.float32) + np.float32(0.5) - np.float32(res / 2)) ** 2
    yz = ax[:, None] + ax[None, :]
    out = []
    for b, s in enumerate(scales):
        r = np.float32(0.45 * res * s)
        for x in range(res):
            d = np.sqrt(ax[x] + yz, dtype=np.float32)
            y, z = np.nonzero((d > r - np.float32(1.0)) & (d <= r))
            if y.size:
                out.append(np.stack([np.full_like(y, b), np.full_like(y, x), y, z], axis=1))
    if not out:
        return np.zeros((0, 4), dtype=np.int32)
    return np.ascontiguousarray(np.concatenate(out, axis=0).astype(np.int32))


def make_problem(res: int, ci: int, co: int, dtype: torch.dtype, seed: int = 0, batch: int = 1,
                 scales: Optional[Sequence[float]] = None, ksize: Tuple[int, int, int] = (3, 3, 3)):
    """(coords, feats, weight, bias, shape) on the CPU: feats ~ N(0,1),
    weight ~ N(0,1)/sqrt(V*Ci), bias ~ N(0,1), drawn in fp32 and cast."""
    g = torch.Generator().manual_seed(seed)
    coords = torch.from_numpy(shell_coords(res, batch, scales))
    V = ksize[0] * ksize[1] * ksize[2]
    feats = torch.randn(coords.shape[0], ci, generator=g).to(dtype)
    weight = (torch.randn(co, *ksize, ci, generator=g) / math.sqrt(V * ci)).to(dtype)
    bias = torch.randn(co, generator=g).to(dtype)
    return coords, feats, weight, bias, torch.Size((batch, ci, res, res, res))


def shell_coords_torch(res: int, batch: int = 1, scales: Optional[Sequence[float]] = None, device="cpu",
                       planes_per_chunk: int = 32) -> torch.Tensor:
    """The rows of ``shell_coords`` (same voxels, same order, int32 [N,4]) computed
    with torch on ``device``: a RES=1024 shell takes milliseconds on a GPU where
    the numpy loop takes tens of seconds.  The distance arithmetic is the same
    sequence of float32 operations (add, multiply, correctly rounded square
    root), so the voxel sets are identical, not just close."""
    if scales is None:
        scales = [1.0] * batch
    dev = torch.device(device)
    half = torch.tensor(res / 2, dtype=torch.float32)
    ax = ((torch.arange(res, dtype=torch.float32) + torch.tensor(0.5, dtype=torch.float32) - half) ** 2).to(dev)
    yz = ax[:, None] + ax[None, :]
    out = []
    for b, s in enumerate(scales):
        r = np.float32(0.45 * res * s)
        lo, hi = float(r - np.float32(1.0)), float(r)
        for x0 in range(0, res, planes_per_chunk):
            x1 = min(res, x0 + planes_per_chunk)
            d = torch.sqrt(ax[x0:x1, None, None] + yz[None])
            idx = torch.nonzero((d > lo) & (d <= hi))          # rows (x - x0, y, z) in lexicographic order
            if idx.shape[0]:
                idx[:, 0] += x0
                out.append(torch.cat([torch.full((idx.shape[0], 1), b, dtype=idx.dtype, device=dev), idx], dim=1).to(torch.int32))
    if not out:
        return torch.zeros((0, 4), dtype=torch.int32, device=dev)
    return torch.cat(out, dim=0).contiguous()
