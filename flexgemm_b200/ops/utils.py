"""Host helpers shared by the ops."""
from typing import Tuple

import torch

from .. import _cabi


def hashmap_key_bits(spatial_size) -> int:
    """32-bit keys while B*W*H*D < 2^32, else 64-bit -- the rule of
    init_hashmap in the reference (flex_gemm/ops/utils.py:4-19)."""
    N, C, W, H, D = [int(s) for s in spatial_size]
    vol = N * W * H * D
    if vol < 2 ** 32:
        return 32
    if vol < 2 ** 64:
        return 64
    raise ValueError(f"The spatial size is too large to fit in a hashmap. Get volumn {vol} > 2^64.")


def init_hashmap(spatial_size, hashmap_size: int, device, with_values: bool = True):
    """The reference's table allocation (flex_gemm/ops/utils.py:4-19): keys of
    ``hashmap_size`` slots filled with all ones -- uint32 while B*W*H*D < 2^32,
    else uint64 -- and, with ``with_values``, an uninitialised uint32 value
    tensor.  Returns ``(hashmap_keys, hashmap_vals)`` or ``hashmap_keys``; these are
    what ``kernels.cuda.hashmap_insert*`` / ``hashmap_lookup*`` take."""
    dtype = torch.uint32 if hashmap_key_bits(spatial_size) == 32 else torch.uint64
    hashmap_keys = torch.full((int(hashmap_size),), torch.iinfo(dtype).max, dtype=dtype, device=device)
    if with_values:
        return hashmap_keys, torch.empty((int(hashmap_size),), dtype=torch.uint32, device=device)
    return hashmap_keys


def init_table(spatial_size, hashmap_size: int, device) -> Tuple[torch.Tensor, int]:
    """Storage for the library's own packed coordinate table of ``hashmap_size``
    slots, as the neighbour-map and grid-sample kernels use it: ``(table,
    key_bits)``.  One opaque buffer (key and row share a 64-bit slot for 32-bit
    keys); the kernels clear it themselves, and it never reaches the caller --
    the reference drops its table after the map is built as well
    (flex_gemm/ops/spconv/submanifold_conv3d.py:57-71)."""
    key_bits = hashmap_key_bits(spatial_size)
    nbytes = _cabi.check_size(_cabi.lib().fgb_hash_table_bytes(int(hashmap_size), key_bits), "fgb_hash_table_bytes")
    table = torch.empty((max(nbytes, 8) + 7) // 8, dtype=torch.int64, device=device)
    return table, key_bits
