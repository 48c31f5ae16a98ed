"""``grid_sample_3d``: features of a sparse voxel grid sampled at arbitrary
points, nearest or trilinear, with the gradient w.r.t. the features.  Names,
arguments and results follow flex_gemm/ops/grid_sample/grid_sample.py:8-212;
the bodies are calls into ``flexgemm_b200.kernels.cuda``."""
from typing import Tuple

import torch
from torch.autograd import Function

from .. import grid_sample, utils
from ... import kernels


def _check(feats, coords, query_pts):
    assert feats.dim() == 2, f"Features must be of shape [N, C], got {feats.shape}"
    assert coords.dim() == 2 and coords.shape[1] == 4, f"Coords must be of shape [N, 4], got {coords.shape}"
    assert query_pts.dim() == 3 and query_pts.shape[2] == 3, f"Query points must be of shape [B, L, 3], got {query_pts.shape}"
    assert feats.shape[0] == coords.shape[0], "Number of features must match number of coordinates"
    if not feats.is_cuda:
        raise NotImplementedError("flexgemm_b200 kernels need CUDA tensors")
    assert feats.shape[1] % 4 == 0, "Channel count must be a multiple of 4"


def _table_for(coords: torch.Tensor, shape):
    C, W, H, D = [int(s) for s in shape[-4:]]
    n = coords.shape[0]
    slots = max(int(grid_sample.HASHMAP_RATIO * n), n, 1)
    table, key_bits = utils.init_table(shape, slots, coords.device)
    status = kernels.cuda.table_insert_3d_idx_as_val(table, key_bits, slots, coords.int().contiguous(), W, H, D)
    return table, key_bits, slots, status, (W, H, D)


class GridSample3dFunction(Function):
    @staticmethod
    def _nearest_fwd(ctx, feats: torch.Tensor, coords: torch.Tensor, shape: torch.Size, query_pts: torch.Tensor) -> torch.Tensor:
        """grid_sample.py:10-53: the feature of the voxel that contains each point, zeros where there is none."""
        _check(feats, coords, query_pts)
        B, L = query_pts.shape[:2]
        table, key_bits, slots, status, (W, H, D) = _table_for(coords, shape)
        indices = kernels.cuda.grid_sample_neighbor_map(table, key_bits, slots, query_pts.float().contiguous(), W, H, D, False)
        out = kernels.cuda.indice_weighted_sum_fwd(feats.contiguous(), indices.view(-1, 1), None).view(B, L, feats.shape[1])
        kernels.cuda.raise_for_status(int(status.item()))
        ctx.save_for_backward(indices)
        ctx.weight = None
        ctx.N = coords.shape[0]
        return out

    @staticmethod
    def _trilinear_fwd(ctx, feats: torch.Tensor, coords: torch.Tensor, shape: torch.Size, query_pts: torch.Tensor) -> torch.Tensor:
        """grid_sample.py:77-123: trilinear blend of the (up to eight) existing voxels around each point, weights
        normalised over the voxels that exist."""
        _check(feats, coords, query_pts)
        B, L = query_pts.shape[:2]
        table, key_bits, slots, status, (W, H, D) = _table_for(coords, shape)
        indices, weight = kernels.cuda.grid_sample_neighbor_map(table, key_bits, slots, query_pts.float().contiguous(), W, H, D, True)
        out = kernels.cuda.indice_weighted_sum_fwd(feats.contiguous(), indices.view(-1, 8), weight.view(-1, 8)).view(B, L, feats.shape[1])
        kernels.cuda.raise_for_status(int(status.item()))
        ctx.save_for_backward(indices, weight)
        ctx.weight = True
        ctx.N = coords.shape[0]
        return out

    @staticmethod
    def _bwd(ctx, grad_output: torch.Tensor) -> Tuple[torch.Tensor, None, None, None, None]:
        """grid_sample.py:55-75, 125-146: scatter-add of the (weighted) output gradient rows."""
        if ctx.weight is None:
            (indices,) = ctx.saved_tensors
            idx, w = indices.view(-1, 1), None
        else:
            indices, weight = ctx.saved_tensors
            idx, w = indices.view(-1, 8), weight.view(-1, 8)
        C = grad_output.shape[-1]
        g32 = kernels.cuda.indice_weighted_sum_bwd(grad_output.reshape(-1, C).contiguous(), idx, w, ctx.N)
        return g32.to(grad_output.dtype), None, None, None, None

    @staticmethod
    def forward(ctx, feats: torch.Tensor, coords: torch.Tensor, shape: torch.Size, grid: torch.Tensor, mode: str = "trilinear") -> torch.Tensor:
        assert mode in ["nearest", "trilinear"], "Invalid interpolation mode"
        ctx.mode = mode
        if mode == "nearest":
            return GridSample3dFunction._nearest_fwd(ctx, feats, coords, shape, grid)
        return GridSample3dFunction._trilinear_fwd(ctx, feats, coords, shape, grid)

    @staticmethod
    def backward(ctx, grad_output: torch.Tensor):
        if ctx.needs_input_grad[0]:
            return GridSample3dFunction._bwd(ctx, grad_output)
        return None, None, None, None, None


def grid_sample_3d(feats: torch.Tensor, coords: torch.Tensor, shape: torch.Size, grid: torch.Tensor, mode: str = "trilinear") -> torch.Tensor:
    """Samples the sparse tensor at the given points.

    Args:
        feats: [N, C] features (float16, bfloat16 or float32, CUDA; C a multiple of 4).
        coords: [N, 4] int32 coordinates (b, x, y, z).
        shape: shape of the dense tensor; its last four entries are (C, W, H, D).
        grid: [B, L, 3] query points in voxel units (voxel (x, y, z) covers [x, x+1) x [y, y+1) x [z, z+1)).
        mode: "nearest" or "trilinear".

    Returns:
        [B, L, C] sampled features.
    """
    return GridSample3dFunction.apply(feats, coords, shape, grid, mode)
