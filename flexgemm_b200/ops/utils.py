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


def init_hashmap(spatial_size, hashmap_size: int, device) -> Tuple[torch.Tensor, int]:
    """Storage for a coordinate hash table of ``hashmap_size`` slots.

    Returns ``(table, key_bits)``.  The table is one opaque byte buffer (its
    layout is private to the CUDA library, which also clears it), unlike the
    reference's separate key/value tensors."""
    key_bits = hashmap_key_bits(spatial_size)
    nbytes = _cabi.check_size(_cabi.lib().fgb_hash_table_bytes(int(hashmap_size), key_bits), "fgb_hash_table_bytes")
    table = torch.empty((max(nbytes, 8) + 7) // 8, dtype=torch.int64, device=device)
    return table, key_bits
