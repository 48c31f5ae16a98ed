"""Sample-sharded data parallelism for the submanifold conv.

A submanifold convolution never couples voxels of different batch indices
(the hash key includes ``b``), so whole samples are independent units: each
rank takes a subset of the samples, re-bases their batch index, builds its own
neighbour cache and runs fprop / dgrad locally.  The one exchange step is the
sum of the weight (and bias) gradient, done as ONE all-reduce of an fp32 buffer
``[Co*V*Ci + Co]`` -- NCCL over NVLink on GPUs.  Outputs and feature gradients
stay sharded.  The reference has no multi-GPU path; this is an addition.
"""
import os
from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


def assign_samples(voxel_counts: Sequence[int], world_size: int) -> List[List[int]]:
    """Longest-processing-time assignment of samples to ranks by voxel count.
    Deterministic: ties go to the lower sample index / lower rank."""
    order = sorted(range(len(voxel_counts)), key=lambda i: (-int(voxel_counts[i]), i))
    loads = [0] * world_size
    out: List[List[int]] = [[] for _ in range(world_size)]
    for i in order:
        r = min(range(world_size), key=lambda k: (loads[k], k))
        out[r].append(i)
        loads[r] += int(voxel_counts[i])
    for lst in out:
        lst.sort()
    return out


def load_balance_bound(voxel_counts: Sequence[int], world_size: int) -> float:
    """Best possible speed-up over one GPU for this assignment: sum / max rank load."""
    parts = assign_samples(voxel_counts, world_size)
    loads = [sum(int(voxel_counts[i]) for i in p) for p in parts]
    return sum(loads) / max(max(loads), 1)


def sample_ranges(coords: torch.Tensor, batch: int) -> List[Tuple[int, int]]:
    """Row range of each sample; ``coords`` must be grouped by batch index in
    ascending order (true for lexicographically sorted coordinates)."""
    b = coords[:, 0].contiguous()
    if b.numel() > 1 and not bool((b[1:] >= b[:-1]).all()):
        raise ValueError("coords must be sorted by batch index to be sharded by sample")
    bounds = torch.searchsorted(b, torch.arange(batch + 1, dtype=b.dtype, device=b.device)).tolist()
    return [(bounds[i], bounds[i + 1]) for i in range(batch)]


def local_shard(coords: torch.Tensor, feats: Optional[torch.Tensor], shape, rank: int, world_size: int):
    """Rows of this rank: ``(local_coords, local_feats, local_shape, rows)`` where
    ``rows`` are the global row indices (int64) in local order and the batch
    index of ``local_coords`` is re-based to 0..k-1."""
    B, C, W, H, D = [int(s) for s in shape]
    ranges = sample_ranges(coords, B)
    mine = assign_samples([e - s for s, e in ranges], world_size)[rank]
    rows, lc = [], []
    for k, i in enumerate(mine):
        s, e = ranges[i]
        rows.append(torch.arange(s, e, device=coords.device))
        c = coords[s:e].clone()
        c[:, 0] = k
        lc.append(c)
    if rows:
        rows_t = torch.cat(rows)
        coords_l = torch.cat(lc).contiguous()
    else:
        rows_t = torch.zeros(0, dtype=torch.int64, device=coords.device)
        coords_l = coords[:0].contiguous()
    feats_l = feats[rows_t].contiguous() if feats is not None else None
    return coords_l, feats_l, torch.Size((max(len(mine), 1), C, W, H, D)), rows_t


# SMs left to the all-reduce of the parameter gradients while dgrad runs (FGB_ALLREDUCE_SMS overrides).  Off by
# default: measured on B200 with NCCL 2.28 it does not pay (2 GPUs: 0.784 ms/step with 0, 0.786 with 8 or 16, 0.831 with
# 32 SMs left over; 8 GPUs: 0.787 with 0, 0.793 with 16) -- NCCL's kernel gets onto the SMs beside the dgrad CTAs.
ALLREDUCE_SMS = int(os.environ.get("FGB_ALLREDUCE_SMS", "0"))


def allreduce_param_grads(gw32: torch.Tensor, gb32: Optional[torch.Tensor], group=None, async_op: bool = False):
    """Sum the fp32 weight (and bias) gradient over the ranks with a single
    all-reduce of one flat buffer; returns views of the reduced buffer (and,
    with ``async_op``, the work handle to wait on before they are read -- None
    when there is nothing to reduce)."""
    nw = gw32.numel()
    flat = torch.empty(nw + (gb32.numel() if gb32 is not None else 0), dtype=torch.float32, device=gw32.device)
    flat[:nw].copy_(gw32.reshape(-1))
    if gb32 is not None:
        flat[nw:].copy_(gb32.reshape(-1))
    work = None
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        work = dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group, async_op=async_op)
    views = (flat[:nw].view_as(gw32), (flat[nw:].view_as(gb32) if gb32 is not None else None))
    return (*views, work) if async_op else views


def sharded_backward(grad_out: torch.Tensor, feats: torch.Tensor, cache, weight: torch.Tensor, bias: Optional[torch.Tensor],
                     group=None, local_grads: Optional[Callable] = None, want_input_grad: bool = True):
    """Backward of the local shard with the parameter gradients summed over the
    ranks.  Returns ``(grad_feats_local, grad_weight, grad_bias)``; the parameter
    gradients are identical on every rank and have the weight's dtype and
    ``[Co, Kw, Kh, Kd, Ci]`` shape.  ``local_grads`` replaces the CUDA kernels in
    host-side tests."""
    Co, Kw, Kh, Kd, Ci = weight.shape
    V = Kw * Kh * Kd
    w = weight.reshape(Co, V, Ci)
    grad_in = None
    if local_grads is None:
        from .kernels import cuda as K
        # One fp32 buffer [Co*V*Ci (+ Co)] is what travels: the split-K reduction and the bias reduction write their
        # fp32 results straight into it, NCCL sums it in place, and one cast kernel turns all of it into the weight dtype.
        nw = Co * V * Ci
        flat = torch.empty(nw + (Co if bias is not None else 0), dtype=torch.float32, device=grad_out.device)
        gw32 = flat[:nw].view(Co, V, Ci)
        gb32 = flat[nw:] if bias is not None else None
        join = None
        if bias is not None:  # small reduction: runs beside the conv kernels on a side stream
            _, _, join = K.bias_grad_overlapped(grad_out, want_f32=True, want_dtype=False, out_f32=gb32)
        # parameter gradients first, so that their all-reduce travels while the input gradient is computed
        K.conv_wgrad(grad_out, feats, cache["valid_signal_i"], cache["valid_signal_o"], cache["valid_signal_seg"], want_f32=True,
                     want_dtype=False, block_offsets=getattr(cache, "pair_block_offsets", None), out_f32=flat[:nw])
        if join is not None:
            join()
        work = None
        if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
            work = dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group, async_op=True)
        if want_input_grad:
            tile = K.conv_tile_rows()
            # the dgrad CTAs fill their SMs: leave the all-reduce a few, or it would only start when dgrad ends
            reserve = ALLREDUCE_SMS if work is not None else 0
            prev = K.set_conv_cta_limit(max(K.sm_count(grad_out.device) - reserve, 1)) if reserve > 0 else None
            try:
                grad_in = K.conv_dgrad(grad_out, w, cache["neighbor_map"], cache["sorted_idx"], cache.tile_masks(tile),
                                       cache.block_order(tile))
            finally:
                if prev is not None:
                    K.set_conv_cta_limit(prev)
        if work is not None:
            work.wait()
        if weight.dtype != torch.float32:
            cast = K.cast_from_f32(flat, weight.dtype)   # weight and bias gradient in one launch
            gw = cast[:nw].view(Co, V, Ci)
            gb = cast[nw:] if bias is not None else None
        else:
            gw, gb = gw32, gb32
        return grad_in, gw.reshape(Co, Kw, Kh, Kd, Ci), gb
    else:
        grad_in, gw32, gb32 = local_grads(grad_out, feats, cache, w, bias is not None)
        gw32, gb32 = allreduce_param_grads(gw32, gb32, group)
    if gw32.is_cuda and weight.dtype != torch.float32:
        from .kernels import cuda as K
        gw = K.cast_from_f32(gw32, weight.dtype)
        gb = K.cast_from_f32(gb32, weight.dtype) if gb32 is not None else None
    else:
        gw = gw32.to(weight.dtype)
        gb = gb32.to(weight.dtype) if gb32 is not None else None
    return grad_in, gw.reshape(Co, Kw, Kh, Kd, Ci), gb
