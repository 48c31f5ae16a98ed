"""``sparse_conv3d`` -- generic (strided / padded / dilated) sparse convolution
and its autograd function on the sm_100a kernels.  Public names, argument
order, cache attribute names and exception classes follow
flex_gemm/ops/spconv/sparse_conv3d.py (line ranges cited per function); the
bodies are calls into ``flexgemm_b200.kernels.cuda``.

The forward pass runs the masked implicit GEMM over the forward map
``neighbor_map`` [L, V]; the input gradient runs the same kernel over the
backward map ``neighbor_map_bwd`` [M, V] (offset v pairs with weight slot v);
the weight gradient runs over the pair lists of the forward map."""
from typing import Optional, Tuple

import torch
from torch.autograd import Function

from . import Algorithm
from .. import spconv, utils
from ... import kernels
from .submanifold_conv3d import _MASKED, _gather_rows


class SparseConv3dNeighborCache:
    """Attribute bag (sparse_conv3d.py:9-56).  ``neighbor_map`` [L,V] and
    ``neighbor_map_bwd`` [M,V] uint32 (the latter None for an inference cache);
    for the implicit-GEMM algorithms also ``gray_code`` / ``sorted_idx`` of the
    forward map, the pair lists ``valid_signal_i/o/seg`` when built for
    training, and ``gray_code_bwd`` / ``sorted_idx_bwd`` of the backward map."""

    def __init__(self, **kwargs):
        for k, v in kwargs.items():
            setattr(self, k, v)

    def __getitem__(self, key):
        return getattr(self, key, None)

    def __setitem__(self, key, value):
        setattr(self, key, value)

    def __contains__(self, key):
        return hasattr(self, key)

    # ---- forward map
    def tile_masks(self, block_size: int) -> torch.Tensor:
        name = f"tile_masks_{block_size}"
        if not hasattr(self, name):
            setattr(self, name, kernels.cuda.tile_masks(self["gray_code"], self["sorted_idx"], block_size))
        return getattr(self, name)

    def block_order(self, block_size: int) -> torch.Tensor:
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

    # ---- backward map
    def _ensure_bwd_order(self):
        """gray code and sorted order of the backward map.  The reference derives
        them only for strided convs or caller-given output coordinates and runs
        the unmasked kernel otherwise (sparse_conv3d.py:192-210); the masked
        kernel is used for every case here, so they are derived on first use."""
        if not hasattr(self, "sorted_idx_bwd"):
            gray, binary = kernels.cuda.gray_code_from_map(self["neighbor_map_bwd"])
            self["gray_code_bwd"] = gray
            self["sorted_idx_bwd"] = kernels.cuda.sorted_idx_from_binary(binary, self["neighbor_map_bwd"].shape[1])

    def tile_masks_bwd(self, block_size: int) -> torch.Tensor:
        name = f"tile_masks_bwd_{block_size}"
        if not hasattr(self, name):
            self._ensure_bwd_order()
            setattr(self, name, kernels.cuda.tile_masks(self["gray_code_bwd"], self["sorted_idx_bwd"], block_size))
        return getattr(self, name)

    def block_order_bwd(self, block_size: int) -> torch.Tensor:
        name = f"block_order_bwd_{block_size}"
        if not hasattr(self, name):
            setattr(self, name, kernels.cuda.block_schedule(self.tile_masks_bwd(block_size)))
        return getattr(self, name)

    def compute_kernel_idx_bwd(self, block_size: int):
        vk, seg = kernels.cuda.valid_kernel(self.tile_masks_bwd(block_size))
        self[f"valid_kernel_bwd_{block_size}"] = vk
        self[f"valid_kernel_bwd_seg_{block_size}"] = seg

    def valid_kernel_bwd_callback(self, block_size: int) -> torch.Tensor:
        if not hasattr(self, f"valid_kernel_bwd_{block_size}"):
            self.compute_kernel_idx_bwd(block_size)
        return self[f"valid_kernel_bwd_{block_size}"]

    def valid_kernel_bwd_seg_callback(self, block_size: int) -> torch.Tensor:
        if not hasattr(self, f"valid_kernel_bwd_seg_{block_size}"):
            self.compute_kernel_idx_bwd(block_size)
        return self[f"valid_kernel_bwd_seg_{block_size}"]


def _out_size(W, H, D, kernel_size, stride, padding, dilation):
    return tuple((n + 2 * p - d * (k - 1) - 1) // s + 1
                 for n, k, s, p, d in zip((W, H, D), kernel_size, stride, padding, dilation))


class SparseConv3dFunction(Function):
    @staticmethod
    def _get_output_coords(coords: torch.Tensor, shape: torch.Size, kernel_size: Tuple[int, int, int], stride: Tuple[int, int, int],
                           padding: Tuple[int, int, int], dilation: Tuple[int, int, int]) -> torch.Tensor:
        """Distinct output voxels, sorted by the key of ``spconv.SERIALIZATION_MODE``
        (sparse_conv3d.py:61-97).  Both values of ``spconv.OUT_COORD_ALGO`` run the
        same hash-set kernel (they differ only in how the reference finds the
        distinct voxels, not in the result)."""
        assert coords.is_contiguous(), "Coords should be contiguous"
        assert coords.dtype in [torch.int32], "Unsupported coords dtype. Expect int32"
        if not coords.is_cuda:
            raise NotImplementedError("CPU version is not implemented")
        if spconv.OUT_COORD_ALGO not in (spconv.SparseConv3dOutCoordAlgorithm.HASHMAP,
                                         spconv.SparseConv3dOutCoordAlgorithm.EXPAND_UNIQUE):
            raise ValueError(f"Unsupported output coordinate algorithm {spconv.OUT_COORD_ALGO}")
        if spconv.SERIALIZATION_MODE not in (0, 1, 2):
            raise RuntimeError("Unsupported serialize mode.")
        return kernels.cuda.sparse_out_coords(coords, shape, kernel_size, stride, padding, dilation,
                                              spconv.OUT_COORD_HASHMAP_RATIO, spconv.SERIALIZATION_MODE)

    @staticmethod
    def _get_output_coords_torch(coords: torch.Tensor, shape: torch.Size, kernel_size: Tuple[int, int, int],
                                 stride: Tuple[int, int, int], padding: Tuple[int, int, int],
                                 dilation: Tuple[int, int, int]) -> torch.Tensor:
        """Library-only construction (expand, filter, ``torch.unique``): rows in
        lexicographic (b, x, y, z) order, i.e. serialisation mode BXYZ
        (sparse_conv3d.py:99-131)."""
        _, _, W, H, D = [int(s) for s in shape]
        Wo, Ho, Do = _out_size(W, H, D, kernel_size, stride, padding, dilation)
        c = coords.to(torch.int64)
        rows = []
        for kx in range(kernel_size[0]):
            for ky in range(kernel_size[1]):
                for kz in range(kernel_size[2]):
                    x = c[:, 1] + padding[0] - kx * dilation[0]
                    y = c[:, 2] + padding[1] - ky * dilation[1]
                    z = c[:, 3] + padding[2] - kz * dilation[2]
                    ok = (x % stride[0] == 0) & (y % stride[1] == 0) & (z % stride[2] == 0)
                    x, y, z = x // stride[0], y // stride[1], z // stride[2]
                    ok &= (x >= 0) & (x < Wo) & (y >= 0) & (y < Ho) & (z >= 0) & (z < Do)
                    rows.append(torch.stack([c[:, 0], x, y, z], dim=1)[ok])
        cand = torch.cat(rows, dim=0) if rows else c[:0]
        return torch.unique(cand, dim=0).to(torch.int32)

    @staticmethod
    def _compute_neighbor_cache(coords: torch.Tensor, out_coords: torch.Tensor, shape: torch.Size, kernel_size: Tuple[int, int, int],
                                stride: Tuple[int, int, int], padding: Tuple[int, int, int], dilation: Tuple[int, int, int],
                                needs_grad: bool, is_out_coords_given: bool = False) -> SparseConv3dNeighborCache:
        """Hash the input voxels, look up the K^3 taps of every output voxel and
        derive the masked-GEMM metadata (sparse_conv3d.py:133-226)."""
        assert coords.is_contiguous(), "Coords should be contiguous"
        assert coords.dtype in [torch.int32], "Unsupported coords dtype. Expect int32"
        if spconv.ALGORITHM not in spconv._ALL_ALGORITHMS:
            raise ValueError(f"Unsupported algorithm {spconv.ALGORITHM}")
        if not coords.is_cuda:
            raise NotImplementedError("CPU version of hashmap is not implemented")
        assert out_coords.is_contiguous() and out_coords.dtype == torch.int32, "Output coords should be contiguous int32"
        V = kernel_size[0] * kernel_size[1] * kernel_size[2]
        assert V <= 32, "Currently, the max kernel volume is 32 because kernel mask is encoded as uint32"
        m = coords.shape[0]
        slots = max(int(spconv.HASHMAP_RATIO * m), m, 1)
        table, key_bits = utils.init_table(shape, slots, coords.device)
        built = kernels.cuda.sparse_build_neighbor_map(coords, out_coords, shape, kernel_size, stride, padding, dilation, table,
                                                       key_bits, slots, needs_grad)
        if spconv.ALGORITHM == Algorithm.EXPLICIT_GEMM:
            kernels.cuda.raise_for_status(int(built["meta"][-1].item()))
            return SparseConv3dNeighborCache(neighbor_map=built["neighbor_map"], neighbor_map_bwd=built["neighbor_map_bwd"])

        if needs_grad:
            # one host round trip: pair count + the build's status word, overlapped with the sort
            meta_host, copied = kernels.cuda.fetch_meta_async(built["meta"])
        sorted_idx = kernels.cuda.sorted_idx_from_binary(built["binary_code"], V)
        cache = SparseConv3dNeighborCache(neighbor_map=built["neighbor_map"], neighbor_map_bwd=built["neighbor_map_bwd"],
                                          gray_code=built["gray_code"], sorted_idx=sorted_idx)
        if needs_grad:
            copied.synchronize()
            kernels.cuda.raise_for_status(int(meta_host[-1]))
            seg = built["valid_signal_seg"]
            vs_i, vs_o = kernels.cuda.valid_signal(built["neighbor_map"], built["gray_code"], built["block_offsets"], seg,
                                                   int(meta_host[V]))
            cache["valid_signal_seg"] = seg
            cache["valid_signal_i"] = vs_i
            cache["valid_signal_o"] = vs_o
            cache["pair_block_offsets"] = built["block_offsets"]   # lets wgrad walk the pair lists in shared row bands
            if any(s != 1 for s in stride) or is_out_coords_given:
                cache._ensure_bwd_order()   # the cases in which the reference also sorts the backward map
        else:
            cache["build_status"] = built["meta"][-1:]
        return cache

    @staticmethod
    def _compute_neighbor_cache_torch(coords: torch.Tensor, out_coords: torch.Tensor, shape: torch.Size,
                                      kernel_size: Tuple[int, int, int], stride: Tuple[int, int, int], padding: Tuple[int, int, int],
                                      dilation: Tuple[int, int, int], needs_grad: bool) -> SparseConv3dNeighborCache:
        """Library-only construction of both maps (sort + searchsorted) with 64-bit
        keys; same result as sparse_conv3d.py:228-281."""
        assert spconv.ALGORITHM == Algorithm.EXPLICIT_GEMM, "Only explicit_gemm is supported for torch implementation"
        _, _, W, H, D = [int(s) for s in shape]
        m, n = coords.shape[0], out_coords.shape[0]
        V = kernel_size[0] * kernel_size[1] * kernel_size[2]
        c, o = coords.to(torch.int64), out_coords.to(torch.int64)
        key = ((c[:, 0] * W + c[:, 1]) * H + c[:, 2]) * D + c[:, 3]
        skey, order = torch.sort(key)
        nbr = torch.full((n, V), 0xFFFFFFFF, dtype=torch.int64, device=coords.device)
        bwd = torch.full((m, V), 0xFFFFFFFF, dtype=torch.int64, device=coords.device) if needs_grad else None
        rows = torch.arange(n, device=coords.device)
        v = 0
        for kx in range(kernel_size[0]):
            for ky in range(kernel_size[1]):
                for kz in range(kernel_size[2]):
                    x = o[:, 1] * stride[0] - padding[0] + kx * dilation[0]
                    y = o[:, 2] * stride[1] - padding[1] + ky * dilation[1]
                    z = o[:, 3] * stride[2] - padding[2] + kz * dilation[2]
                    ok = (x >= 0) & (x < W) & (y >= 0) & (y < H) & (z >= 0) & (z < D)
                    if m and n:
                        nkey = ((o[:, 0] * W + x) * H + y) * D + z
                        pos = torch.searchsorted(skey, nkey).clamp_(0, m - 1)
                        ok &= skey[pos] == nkey
                        src = order[pos]
                        nbr[:, v] = torch.where(ok, src, nbr[:, v])
                        if needs_grad:
                            bwd[src[ok], v] = rows[ok]
                    v += 1
        return SparseConv3dNeighborCache(neighbor_map=nbr.to(torch.uint32),
                                         neighbor_map_bwd=bwd.to(torch.uint32) if needs_grad else None)

    @staticmethod
    def _sparse_conv_forward(feats: torch.Tensor, neighbor_cache: SparseConv3dNeighborCache, weight: torch.Tensor,
                             bias: Optional[torch.Tensor] = None) -> torch.Tensor:
        """sparse_conv3d.py:283-350."""
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
    def _sparse_conv_backward(grad_output: torch.Tensor, feats: torch.Tensor, neighbor_cache: SparseConv3dNeighborCache,
                              weight: torch.Tensor, bias: Optional[torch.Tensor] = None
                              ) -> Tuple[Optional[torch.Tensor], Optional[torch.Tensor], Optional[torch.Tensor]]:
        """sparse_conv3d.py:352-451."""
        Co, Kw, Kh, Kd, Ci = weight.shape
        V = Kd * Kh * Kw
        grad_input = grad_weight = grad_bias = None
        if spconv.ALGORITHM == Algorithm.EXPLICIT_GEMM:
            if feats.requires_grad:
                col = _gather_rows(grad_output, neighbor_cache["neighbor_map_bwd"])
                grad_input = torch.mm(col, weight.reshape(Co, V, Ci).transpose(0, 1).reshape(V * Co, Ci))
            if weight.requires_grad:
                col = _gather_rows(feats, neighbor_cache["neighbor_map"])
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
                neighbor_cache._ensure_bwd_order()
                grad_input = kernels.cuda.conv_dgrad(grad_output, w, neighbor_cache["neighbor_map_bwd"], neighbor_cache["sorted_idx_bwd"],
                                                     neighbor_cache.tile_masks_bwd(tile), neighbor_cache.block_order_bwd(tile),
                                                     mirror=False)
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
                neighbor_cache: Optional[SparseConv3dNeighborCache], weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
                out_coords: Optional[torch.Tensor] = None, stride: Tuple[int, int, int] = (1, 1, 1),
                padding: Tuple[int, int, int] = (0, 0, 0), dilation: Tuple[int, int, int] = (1, 1, 1)
                ) -> Tuple[torch.Tensor, torch.Tensor, SparseConv3dNeighborCache]:
        """sparse_conv3d.py:453-483."""
        Co, Kw, Kh, Kd, Ci = weight.shape
        assert feats.shape[-1] == Ci, f"Input channels ({feats.shape[-1]}) should match weight channels ({Ci})"
        need_grad = any(ctx.needs_input_grad)
        given = out_coords is not None
        if out_coords is None:
            out_coords = SparseConv3dFunction._get_output_coords(coords, shape, (Kw, Kh, Kd), stride, padding, dilation)
        if neighbor_cache is None:
            neighbor_cache = SparseConv3dFunction._compute_neighbor_cache(coords, out_coords, shape, (Kw, Kh, Kd), stride, padding,
                                                                          dilation, need_grad, given)
        output = SparseConv3dFunction._sparse_conv_forward(feats, neighbor_cache, weight, bias)
        ctx.save_for_backward(feats, weight, bias)
        ctx.neighbor_cache = neighbor_cache
        ctx.mark_non_differentiable(out_coords)
        return output, out_coords, neighbor_cache

    @staticmethod
    def backward(ctx, grad_output: torch.Tensor, _, __):
        """sparse_conv3d.py:485-499; additionally accepts ``bias=None``."""
        feats, weight, bias = ctx.saved_tensors
        feats_r = feats.detach().requires_grad_(ctx.needs_input_grad[0])
        weight_r = weight.detach().requires_grad_(ctx.needs_input_grad[4])
        bias_r = bias.detach().requires_grad_(ctx.needs_input_grad[5]) if bias is not None else None
        grad_input, grad_weight, grad_bias = SparseConv3dFunction._sparse_conv_backward(
            grad_output, feats_r, ctx.neighbor_cache, weight_r, bias_r)
        return grad_input, None, None, None, grad_weight, grad_bias, None, None, None, None


def sparse_conv3d(feats: torch.Tensor, coords: torch.Tensor, shape: torch.Size, weight: torch.Tensor,
                  bias: Optional[torch.Tensor] = None, neighbor_cache: Optional[SparseConv3dNeighborCache] = None,
                  out_coords: Optional[torch.Tensor] = None, stride: Tuple[int, int, int] = (1, 1, 1),
                  padding: Tuple[int, int, int] = (0, 0, 0), dilation: Tuple[int, int, int] = (1, 1, 1)
                  ) -> Tuple[torch.Tensor, torch.Tensor, SparseConv3dNeighborCache]:
    """Sparse convolution for 3D input.

    Args:
        feats: [N, C] input features (float16, bfloat16 or float32, CUDA).
        coords: [N, 4] int32 input coordinates (b, x, y, z).
        shape: shape of the dense input tensor in NCWHD order.
        weight: [Co, Kw, Kh, Kd, Ci] weights.
        bias: optional [Co] bias.
        neighbor_cache: cache returned by an earlier call with the same coordinates and geometry.
        out_coords: optional [M, 4] int32 output coordinates; derived from the input
            coordinates, kernel size, stride, padding and dilation when None.
        stride, padding, dilation: per axis.

    Returns:
        (out_feats [M, Co], out_coords [M, 4], neighbor_cache)
    """
    return SparseConv3dFunction.apply(feats, coords, shape, neighbor_cache, weight, bias, out_coords, stride, padding, dilation)
