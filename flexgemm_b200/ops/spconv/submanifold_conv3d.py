"""``sparse_submanifold_conv3d`` and its autograd function on the sm_100a
kernels.  Public names, argument order, cache attribute names, exception
classes and the ``[Co, Kw, Kh, Kd, Ci]`` weight layout follow
flex_gemm/ops/spconv/submanifold_conv3d.py (the line ranges are cited per
function); the bodies are calls into ``flexgemm_b200.kernels.cuda``."""
from typing import Optional, Tuple

import torch
from torch.autograd import Function

from . import Algorithm
from .. import spconv, utils
from ... import kernels

_MASKED = (Algorithm.IMPLICIT_GEMM, Algorithm.IMPLICIT_GEMM_SPLITK,
           Algorithm.MASKED_IMPLICIT_GEMM, Algorithm.MASKED_IMPLICIT_GEMM_SPLITK)


class SubMConv3dNeighborCache:
    """Attribute bag holding the neighbour map and what was derived from it
    (submanifold_conv3d.py:9-41).  Attributes: ``neighbor_map`` [N,V] uint32,
    ``gray_code`` [N] int32, ``sorted_idx`` [N] int64, and -- when built for
    training -- ``valid_signal_i`` / ``valid_signal_o`` [L] uint32 and
    ``valid_signal_seg`` [V+1] uint32.  Per tile size B, ``tile_masks_B`` (the
    form the kernels consume) and ``valid_kernel_B`` / ``valid_kernel_seg_B``
    (the reference's list form) are computed on first use."""

    def __init__(self, **kwargs):
        for k, v in kwargs.items():
            setattr(self, k, v)

    def __getitem__(self, key):
        return getattr(self, key)

    def __setitem__(self, key, value):
        setattr(self, key, value)

    def __contains__(self, key):
        return hasattr(self, key)

    def tile_masks(self, block_size: int) -> torch.Tensor:
        name = f"tile_masks_{block_size}"
        if not hasattr(self, name):
            setattr(self, name, kernels.cuda.tile_masks(self["gray_code"], self["sorted_idx"], block_size))
        return getattr(self, name)

    def block_order(self, block_size: int) -> torch.Tensor:
        """Pairs of consecutive tiles in descending order of work (the schedule of
        the persistent kernels); computed with the tile masks, once per cache."""
        name = f"block_order_{block_size}"
        if not hasattr(self, name):
            setattr(self, name, kernels.cuda.block_schedule(self.tile_masks(block_size)))
        return getattr(self, name)

    def compute_kernel_idx(self, block_size: int):
        vk, seg = kernels.cuda.valid_kernel(self.tile_masks(block_size))
        self[f"valid_kernel_{block_size}"] = vk
        self[f"valid_kernel_seg_{block_size}"] = seg

    def valid_kernel_callback(self, block_size: int) -> torch.Tensor:
        if not hasattr(self, f"valid_kernel_{block_size}"):
            self.compute_kernel_idx(block_size)
        return self[f"valid_kernel_{block_size}"]

    def valid_kernel_seg_callback(self, block_size: int) -> torch.Tensor:
        if not hasattr(self, f"valid_kernel_seg_{block_size}"):
            self.compute_kernel_idx(block_size)
        return self[f"valid_kernel_seg_{block_size}"]


def _gather_rows(x: torch.Tensor, nbr: torch.Tensor) -> torch.Tensor:
    """[N, V*C] matrix whose (n, v) block is x[nbr[n, v]] or zeros."""
    n, V = nbr.shape
    idx = nbr.reshape(-1).to(torch.int64)
    missing = idx == 0xFFFFFFFF
    padded = torch.cat([x, x.new_zeros(1, x.shape[1])], dim=0)
    return padded[torch.where(missing, torch.full_like(idx, x.shape[0]), idx)].view(n, V * x.shape[1])


class SubMConv3dFunction(Function):
    @staticmethod
    def _compute_neighbor_cache(coords: torch.Tensor, shape: torch.Size, kernel_size: Tuple[int, int, int],
                                dilation: Tuple[int, int, int], needs_grad: bool) -> SubMConv3dNeighborCache:
        """Hash the coordinates, look up the K^3 neighbourhood of every voxel and
        derive the masked-GEMM metadata (submanifold_conv3d.py:45-107)."""
        assert coords.is_contiguous(), "Coords should be contiguous"
        assert coords.dtype in [torch.int32], "Unsupported coords dtype. Expect int32"
        if spconv.ALGORITHM not in spconv._ALL_ALGORITHMS:
            raise ValueError(f"Unsupported algorithm {spconv.ALGORITHM}")
        if not coords.is_cuda:
            raise NotImplementedError("CPU version of hashmap is not implemented")
        V = kernel_size[0] * kernel_size[1] * kernel_size[2]
        assert V <= 32, "Currently, the max kernel volume is 32 because kernel mask is encoded as uint32"
        assert all(int(k) % 2 == 1 for k in kernel_size), "Kernel extents must be odd"
        n = coords.shape[0]
        slots = max(int(spconv.HASHMAP_RATIO * n), n, 1)
        table, key_bits = utils.init_table(shape, slots, coords.device)
        built = kernels.cuda.subm_build_neighbor_map(coords, shape, kernel_size, dilation, table, key_bits, slots)
        if spconv.ALGORITHM == Algorithm.EXPLICIT_GEMM:
            kernels.cuda.raise_for_status(int(built["meta"][-1].item()))
            return SubMConv3dNeighborCache(neighbor_map=built["neighbor_map"])

        if needs_grad:
            # The one host round trip of the build: the pair count sizes the lists, and
            # the same copy brings the build's status word (hash table overflow).  The
            # copy is queued before the sort so that the host wait overlaps the sort.
            meta_host, copied = kernels.cuda.fetch_meta_async(built["meta"])
        sorted_idx = kernels.cuda.sorted_idx_from_binary(built["binary_code"], V)
        cache = SubMConv3dNeighborCache(neighbor_map=built["neighbor_map"], gray_code=built["gray_code"], sorted_idx=sorted_idx)
        if needs_grad:
            copied.synchronize()
            kernels.cuda.raise_for_status(int(meta_host[-1]))
            seg = built["valid_signal_seg"]
            num_pairs = int(meta_host[V])
            vs_i, vs_o = kernels.cuda.valid_signal(built["neighbor_map"], built["gray_code"], built["block_offsets"], seg, num_pairs,
                                                   built["order_flag"])
            cache["valid_signal_seg"] = seg
            cache["valid_signal_i"] = vs_i
            cache["valid_signal_o"] = vs_o
            # not part of the reference's cache: where each 256-row block starts in every offset's pair list, which
            # lets wgrad walk all lists in row bands that share L2
            cache["pair_block_offsets"] = built["block_offsets"]
        else:
            # inference cache: nothing needs the host, so nothing synchronises; an
            # overflowing table would show in this word, readable at any later time
            cache["build_status"] = built["meta"][-1:]
        return cache

    @staticmethod
    def _compute_neighbor_cache_torch(coords: torch.Tensor, shape: torch.Size, kernel_size: Tuple[int, int, int],
                                      dilation: Tuple[int, int, int]) -> SubMConv3dNeighborCache:
        """Library-only construction of the neighbour map (sort + searchsorted),
        usable on any device; same result as submanifold_conv3d.py:109-144 but
        with 64-bit keys, so it has no 2^31 limit."""
        assert spconv.ALGORITHM == Algorithm.EXPLICIT_GEMM, "Only explicit_gemm is supported for torch implementation"
        _, _, W, H, D = [int(s) for s in shape]
        n = coords.shape[0]
        c = coords.to(torch.int64)
        key = ((c[:, 0] * W + c[:, 1]) * H + c[:, 2]) * D + c[:, 3]
        skey, order = torch.sort(key)
        cols = []
        for kx in range(kernel_size[0]):
            for ky in range(kernel_size[1]):
                for kz in range(kernel_size[2]):
                    x = c[:, 1] + (kx - kernel_size[0] // 2) * dilation[0]
                    y = c[:, 2] + (ky - kernel_size[1] // 2) * dilation[1]
                    z = c[:, 3] + (kz - kernel_size[2] // 2) * dilation[2]
                    ok = (x >= 0) & (x < W) & (y >= 0) & (y < H) & (z >= 0) & (z < D)
                    nkey = ((c[:, 0] * W + x) * H + y) * D + z
                    pos = torch.searchsorted(skey, nkey).clamp_(0, max(n - 1, 0))
                    if n:
                        ok &= skey[pos] == nkey
                        cols.append(torch.where(ok, order[pos], torch.full_like(pos, 0xFFFFFFFF)))
                    else:
                        cols.append(pos)
        return SubMConv3dNeighborCache(neighbor_map=torch.stack(cols, dim=1).to(torch.uint32))

    @staticmethod
    def _sparse_submanifold_conv_forward(feats: torch.Tensor, neighbor_cache: SubMConv3dNeighborCache, weight: torch.Tensor,
                                         bias: Optional[torch.Tensor] = None) -> torch.Tensor:
        """submanifold_conv3d.py:146-215."""
        assert feats.is_contiguous(), "Input features should be contiguous"
        Co, Kw, Kh, Kd, Ci = weight.shape
        V = Kd * Kh * Kw
        if spconv.ALGORITHM == Algorithm.EXPLICIT_GEMM:
            col = _gather_rows(feats, neighbor_cache["neighbor_map"])
            w = weight.reshape(Co, V * Ci).t()
            return torch.addmm(bias, col, w) if bias is not None else torch.mm(col, w)
        if spconv.ALGORITHM in _MASKED:
            if not feats.is_cuda:
                raise NotImplementedError("flexgemm_b200 kernels need CUDA tensors")
            assert weight.is_contiguous(), "Matrix weight must be contiguous"
            tile = kernels.cuda.conv_tile_rows()
            return kernels.cuda.conv_fprop(
                feats, weight.reshape(Co, V, Ci), bias.contiguous() if bias is not None else None,
                neighbor_cache["neighbor_map"], neighbor_cache["sorted_idx"], neighbor_cache.tile_masks(tile),
                neighbor_cache.block_order(tile))
        raise ValueError(f"Unsupported algorithm {spconv.ALGORITHM}")

    @staticmethod
    def _sparse_submanifold_conv_backward(grad_output: torch.Tensor, feats: torch.Tensor, neighbor_cache: SubMConv3dNeighborCache,
                                          weight: torch.Tensor, bias: Optional[torch.Tensor] = None
                                          ) -> Tuple[Optional[torch.Tensor], Optional[torch.Tensor], Optional[torch.Tensor]]:
        """submanifold_conv3d.py:217-317.  Gradients are produced for the inputs
        whose ``requires_grad`` is set."""
        Co, Kw, Kh, Kd, Ci = weight.shape
        V = Kd * Kh * Kw
        grad_input = grad_weight = grad_bias = None
        if spconv.ALGORITHM == Algorithm.EXPLICIT_GEMM:
            nbr = neighbor_cache["neighbor_map"]
            if feats.requires_grad:
                col = _gather_rows(grad_output, torch.flip(nbr.view(torch.int32), [1]).view(torch.uint32))
                grad_input = torch.mm(col, weight.reshape(Co, V, Ci).transpose(0, 1).reshape(V * Co, Ci))
            if weight.requires_grad:
                col = _gather_rows(feats, nbr)
                grad_weight = torch.mm(col.t(), grad_output).view(V, Ci, Co).permute(2, 0, 1).contiguous().view(Co, Kw, Kh, Kd, Ci)
            if bias is not None and bias.requires_grad:
                grad_bias = grad_output.sum(dim=0)
            return grad_input, grad_weight, grad_bias
        if spconv.ALGORITHM in _MASKED:
            grad_output = grad_output.contiguous()
            assert feats.is_contiguous(), "Matrix input must be contiguous"
            assert weight.is_contiguous(), "Matrix weight must be contiguous"
            w = weight.reshape(Co, V, Ci)
            join = None
            if bias is not None and bias.requires_grad:   # a small reduction: runs beside the conv kernels
                grad_bias, _, join = kernels.cuda.bias_grad_overlapped(grad_output)
            if feats.requires_grad:
                tile = kernels.cuda.conv_tile_rows()
                grad_input = kernels.cuda.conv_dgrad(grad_output, w, neighbor_cache["neighbor_map"], neighbor_cache["sorted_idx"],
                                                     neighbor_cache.tile_masks(tile), neighbor_cache.block_order(tile))
            if weight.requires_grad:
                gw, _ = kernels.cuda.conv_wgrad(grad_output, feats, neighbor_cache["valid_signal_i"], neighbor_cache["valid_signal_o"],
                                                neighbor_cache["valid_signal_seg"],
                                                block_offsets=getattr(neighbor_cache, "pair_block_offsets", None))
                grad_weight = gw.reshape(Co, Kw, Kh, Kd, Ci)
            if join is not None:
                join()
            return grad_input, grad_weight, grad_bias
        raise ValueError(f"Unsupported algorithm {spconv.ALGORITHM}")

    @staticmethod
    def forward(ctx, feats: torch.Tensor, coords: torch.Tensor, shape: torch.Size,
                neighbor_cache: Optional[SubMConv3dNeighborCache], weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
                dilation: Tuple[int, int, int] = (1, 1, 1)) -> Tuple[torch.Tensor, SubMConv3dNeighborCache]:
        """submanifold_conv3d.py:319-345."""
        Co, Kw, Kh, Kd, Ci = weight.shape
        assert feats.shape[-1] == Ci, f"Input channels ({feats.shape[-1]}) should match weight channels ({Ci})"
        need_grad = any(ctx.needs_input_grad)
        if neighbor_cache is None:
            neighbor_cache = SubMConv3dFunction._compute_neighbor_cache(coords, shape, (Kw, Kh, Kd), dilation, need_grad)
        output = SubMConv3dFunction._sparse_submanifold_conv_forward(feats, neighbor_cache, weight, bias)
        ctx.save_for_backward(feats, weight, bias)
        ctx.neighbor_cache = neighbor_cache
        return output, neighbor_cache

    @staticmethod
    def backward(ctx, grad_output: torch.Tensor, _):
        """submanifold_conv3d.py:347-360; additionally accepts ``bias=None``."""
        feats, weight, bias = ctx.saved_tensors
        # the kernels decide what to compute from requires_grad, as the reference's do
        feats_r = feats.detach().requires_grad_(ctx.needs_input_grad[0])
        weight_r = weight.detach().requires_grad_(ctx.needs_input_grad[4])
        bias_r = bias.detach().requires_grad_(ctx.needs_input_grad[5]) if bias is not None else None
        grad_input, grad_weight, grad_bias = SubMConv3dFunction._sparse_submanifold_conv_backward(
            grad_output, feats_r, ctx.neighbor_cache, weight_r, bias_r)
        return grad_input, None, None, None, grad_weight, grad_bias, None


def sparse_submanifold_conv3d(feats: torch.Tensor, coords: torch.Tensor, shape: torch.Size, weight: torch.Tensor,
                              bias: Optional[torch.Tensor] = None, neighbor_cache: Optional[SubMConv3dNeighborCache] = None,
                              dilation: Tuple[int, int, int] = (1, 1, 1)) -> Tuple[torch.Tensor, SubMConv3dNeighborCache]:
    """Sparse submanifold convolution for 3D input.

    Args:
        feats: [N, C] input features (float16, bfloat16 or float32, CUDA).
        coords: [N, 4] int32 coordinates (b, x, y, z).
        shape: shape of the dense tensor in NCWHD order.
        weight: [Co, Kw, Kh, Kd, Ci] weights.
        bias: optional [Co] bias.
        neighbor_cache: cache returned by an earlier call on the same coordinates;
            built on the fly when None.
        dilation: dilation per axis.

    Returns:
        (output [N, Co], neighbor_cache)
    """
    return SubMConv3dFunction.apply(feats, coords, shape, neighbor_cache, weight, bias, dilation)
