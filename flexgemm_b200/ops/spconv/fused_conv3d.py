"""Submanifold conv with the elementwise work of a residual block fused into the
forward kernel's epilogue:

    out = activation(conv(feats) + bias) + residual

The reference has no such call: its callers run torch kernels between the convs
of a residual stack ([conv, SiLU, conv] + skip).  The conv itself, the cache and
the backward kernels are those of ``sparse_submanifold_conv3d``
(flex_gemm/ops/spconv/submanifold_conv3d.py:319-391); only the epilogue differs.
The result carries the roundings of the unfused sequence (conv result rounded to
the feature dtype, activation in fp32 and rounded, add rounded).

Measured on B200 (N = 39 872 voxels, C = 512, bf16) the fused forward is slower
than conv + a torch elementwise kernel (SiLU: 462 against 345 us; residual: 373
against 341 us): the fused kernel instance spills registers that the plain one
does not.  Use it where one kernel launch matters more than that (CUDA-graph
size, launch-bound small inputs), not for throughput."""
from typing import Optional, Tuple

import torch
from torch.autograd import Function

from .. import spconv
from ... import kernels
from .submanifold_conv3d import _MASKED, SubMConv3dFunction, SubMConv3dNeighborCache

ACTIVATIONS = (None, "silu")


def _silu_grad(preact: torch.Tensor, grad: torch.Tensor) -> torch.Tensor:
    """grad * d silu(y)/dy at y = ``preact``: torch's own one-kernel backward of SiLU."""
    return torch.ops.aten.silu_backward(grad, preact)


class SubMConv3dFusedFunction(Function):
    @staticmethod
    def forward(ctx, feats: torch.Tensor, coords: torch.Tensor, shape: torch.Size,
                neighbor_cache: Optional[SubMConv3dNeighborCache], weight: torch.Tensor, bias: Optional[torch.Tensor],
                dilation: Tuple[int, int, int], activation: Optional[str], residual: Optional[torch.Tensor]):
        if activation not in ACTIVATIONS:
            raise ValueError(f"Unsupported activation {activation!r}")
        if spconv.ALGORITHM not in _MASKED:
            raise NotImplementedError("the fused epilogue exists for the implicit-GEMM algorithms only")
        if not feats.is_cuda:
            raise NotImplementedError("flexgemm_b200 kernels need CUDA tensors")
        assert feats.is_contiguous(), "Input features should be contiguous"
        assert weight.is_contiguous(), "Matrix weight must be contiguous"
        Co, Kw, Kh, Kd, Ci = weight.shape
        assert feats.shape[-1] == Ci, f"Input channels ({feats.shape[-1]}) should match weight channels ({Ci})"
        V = Kw * Kh * Kd
        conv_needs = ctx.needs_input_grad[0] or ctx.needs_input_grad[4] or ctx.needs_input_grad[5]
        if neighbor_cache is None:
            neighbor_cache = SubMConv3dFunction._compute_neighbor_cache(coords, shape, (Kw, Kh, Kd), dilation, conv_needs)
        tile = kernels.cuda.conv_tile_rows()
        # the activation's backward needs the conv result itself: the kernel keeps a copy of it only then
        keep = activation is not None and conv_needs
        out, preact = kernels.cuda.conv_fprop_fused(
            feats, weight.reshape(Co, V, Ci), bias.contiguous() if bias is not None else None,
            neighbor_cache["neighbor_map"], neighbor_cache["sorted_idx"], neighbor_cache.tile_masks(tile),
            neighbor_cache.block_order(tile), activation=activation,
            residual=residual.contiguous() if residual is not None else None, keep_preact=keep)
        ctx.save_for_backward(feats, weight, bias, preact)
        ctx.neighbor_cache = neighbor_cache
        ctx.activation = activation
        return out, neighbor_cache

    @staticmethod
    def backward(ctx, grad_output: torch.Tensor, _):
        feats, weight, bias, preact = ctx.saved_tensors
        grad_output = grad_output.contiguous()
        grad_residual = grad_output if ctx.needs_input_grad[8] else None
        conv_needs = ctx.needs_input_grad[0] or ctx.needs_input_grad[4] or ctx.needs_input_grad[5]
        if not conv_needs:
            return None, None, None, None, None, None, None, None, grad_residual
        g = _silu_grad(preact, grad_output) if ctx.activation == "silu" else grad_output
        feats_r = feats.detach().requires_grad_(ctx.needs_input_grad[0])
        weight_r = weight.detach().requires_grad_(ctx.needs_input_grad[4])
        bias_r = bias.detach().requires_grad_(ctx.needs_input_grad[5]) if bias is not None else None
        grad_input, grad_weight, grad_bias = SubMConv3dFunction._sparse_submanifold_conv_backward(
            g, feats_r, ctx.neighbor_cache, weight_r, bias_r)
        return grad_input, None, None, None, grad_weight, grad_bias, None, None, grad_residual


def sparse_submanifold_conv3d_fused(feats: torch.Tensor, coords: torch.Tensor, shape: torch.Size, weight: torch.Tensor,
                                    bias: Optional[torch.Tensor] = None, neighbor_cache: Optional[SubMConv3dNeighborCache] = None,
                                    dilation: Tuple[int, int, int] = (1, 1, 1), activation: Optional[str] = None,
                                    residual: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, SubMConv3dNeighborCache]:
    """``activation(sparse_submanifold_conv3d(...)) + residual`` in one kernel.

    Args as ``sparse_submanifold_conv3d``, plus
        activation: None or "silu".
        residual: optional [N, Co] tensor of the feature dtype, added after the activation.

    Returns:
        (output [N, Co], neighbor_cache)
    """
    return SubMConv3dFusedFunction.apply(feats, coords, shape, neighbor_cache, weight, bias, dilation, activation, residual)
