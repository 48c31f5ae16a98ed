"""Tensor-level wrappers over the C ABI (``include/flexgemm_b200.h``).

These play the role of the reference's ``flex_gemm.kernels.cuda`` pybind
module (flex_gemm/kernels/cuda/ext.cpp:10-36) and of its Triton wrappers for
the submanifold path: they allocate outputs with torch, pass raw pointers and
the current CUDA stream to the library, and never compute anything themselves.
"""
from typing import Dict, Optional, Tuple

import torch

from .. import _cabi
from . import config

_DTYPES = {torch.float16: _cabi.F16, torch.bfloat16: _cabi.BF16}


def dtype_code(dtype: torch.dtype) -> int:
    if dtype in _DTYPES:
        return _DTYPES[dtype]
    if dtype == torch.float32:
        return _cabi.F32_TF32 if config.allow_tf32 else _cabi.F32_IEEE
    raise TypeError(f"unsupported feature dtype {dtype}: expected float16, bfloat16 or float32")


def _require_cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise NotImplementedError(f"{name} must be a CUDA tensor: flexgemm_b200 has no CPU implementation")


def _ptr(t: Optional[torch.Tensor]) -> int:
    return 0 if t is None or t.numel() == 0 else t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream(device) -> int:
    # the raw handle of torch's current stream on `device`; the direct binding avoids building a Stream object per call
    # (every wrapper here asks for it, a cache build a dozen times)
    if _raw_stream is not None:
        idx = device.index if isinstance(device, torch.device) else device
        return _raw_stream(torch.cuda.current_device() if idx is None else idx)
    return torch.cuda.current_stream(device).cuda_stream


# --------------------------------------------------------------------------
# per-(device, stream) scratch and the device status word
# --------------------------------------------------------------------------
_scratch: Dict[tuple, torch.Tensor] = {}
_status: Dict[int, torch.Tensor] = {}

# Number of this library's own kernels launched so far.  Each wrapper adds the
# number of kernels its C entry point launches.
launch_count = 0


def _count(k: int) -> None:
    global launch_count
    launch_count += k


def workspace(device: torch.device, tag: str, nbytes: int) -> torch.Tensor:
    """A reusable 256-byte aligned scratch buffer of at least ``nbytes`` bytes.
    Buffers are keyed by stream so that work on one stream never shares scratch
    with work on another."""
    key = (device.index, _stream(device), tag)
    buf = _scratch.get(key)
    if buf is None or buf.numel() * 8 < nbytes:
        buf = torch.empty(max(int(nbytes) + 7, 256) // 8, dtype=torch.int64, device=device)
        _scratch[key] = buf
    return buf


def release_workspaces() -> None:
    _scratch.clear()


def status_word(device: torch.device) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _status:
        _status[idx] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status[idx]


def check_status(device: torch.device) -> None:
    """Read (synchronising) and clear the device status word; raise if a kernel
    recorded a soft error."""
    word = status_word(device)
    code = int(word.item())
    _status_pending.pop(_device_index(device), None)
    if code != 0:
        word.zero_()
        raise_for_status(code)


def _device_index(device: torch.device) -> int:
    return device.index if device.index is not None else torch.cuda.current_device()


# device index -> (pinned host word, event recorded after the copy that fills it)
_status_pending: Dict[int, tuple] = {}


def poll_status(device: torch.device) -> None:
    """Non-blocking look at the device status word, called by the conv wrappers
    before they launch.

    A kernel that hits a soft error (a bounded barrier wait that ran out, a full
    hash table) records a code in the word and every later conv kernel on that
    device returns at once while it is set, so the error must reach the caller:
    this function queues a 4-byte copy of the word to pinned host memory and, on
    a later call, once that copy has landed, looks at it.  A non-zero code clears
    the word (so that the calls after the exception run normally) and raises
    ``RuntimeError``.  Nothing here waits for the GPU; the error therefore
    surfaces at the first conv call made after the device has reported it --
    ``check_status`` is the synchronising variant."""
    idx = _device_index(device)
    entry = _status_pending.get(idx)
    if entry is not None:
        host, event = entry
        if not event.query():
            return  # the previous copy is still in flight: look again at the next call
        code = int(host[0])
        del _status_pending[idx]
        if code != 0:
            status_word(device).zero_()
            raise_for_status(code)
    else:
        host = None
    if host is None:
        host = _status_host.get(idx)
        if host is None:
            host = _status_host[idx] = torch.zeros(1, dtype=torch.int32).pin_memory()
    event = torch.cuda.Event()
    host.copy_(status_word(device), non_blocking=True)
    event.record(torch.cuda.current_stream(device))
    _status_pending[idx] = (host, event)


_status_host: Dict[int, torch.Tensor] = {}


# --------------------------------------------------------------------------
# neighbour map and post-processing
# --------------------------------------------------------------------------
_zero_pool: Dict[tuple, list] = {}


def _zeroed_words(device: torch.device, count: int) -> torch.Tensor:
    """``count`` zeroed uint32 words that nothing else uses: a slice of a pool that is zeroed 4096 words at a time, so
    that a cache build does not launch a fill kernel of its own (the slices stay alive with the tensors that view
    them; a pool is dropped when it is used up)."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    key = (idx, _stream(device))      # zeroed on the stream that uses it
    entry = _zero_pool.get(key)
    words = (count + 7) & ~7          # 32-byte slices
    if entry is None or entry[1] + words > entry[0].numel():
        entry = _zero_pool[key] = [torch.zeros(max(4096, words), dtype=torch.uint32, device=device), 0]
    out = entry[0][entry[1]:entry[1] + count]
    entry[1] += words
    return out


def subm_build_neighbor_map(coords: torch.Tensor, shape, ksize, dilation, table: torch.Tensor, key_bits: int,
                            slots: int) -> Dict[str, torch.Tensor]:
    """Hash build + lookup.  Returns neighbor_map [N,V] uint32, gray_code and
    binary_code [N] int32, block_offsets [V*nblk] uint32, valid_signal_seg [V+1]
    uint32 and ``meta`` (uint32 [V+3]: the segment array, the word that is 0 when
    the rows were in key order -- ``order_flag`` -- and this call's own status
    word, so that one device-to-host copy fetches all of them)."""
    _require_cuda(coords, "coords")
    lib = _cabi.lib()
    dev = coords.device
    n = coords.shape[0]
    B, _, W, H, D = [int(s) for s in shape]
    V = int(ksize[0]) * int(ksize[1]) * int(ksize[2])
    nblk = _cabi.check_size(lib.fgb_map_num_blocks(n), "fgb_map_num_blocks")
    meta = _zeroed_words(dev, V + 3)
    out = {
        "neighbor_map": torch.empty((n, V), dtype=torch.uint32, device=dev),
        "gray_code": torch.empty(n, dtype=torch.int32, device=dev),
        "binary_code": torch.empty(n, dtype=torch.int32, device=dev),
        "block_offsets": torch.empty(max(V * nblk, 1), dtype=torch.uint32, device=dev),
        "valid_signal_seg": meta[:V + 1],
        "order_flag": meta[V + 1:V + 2],
        "meta": meta,
    }
    rc = lib.fgb_subm_build_neighbor_map(
        _ptr(coords), n, B, W, H, D, int(ksize[0]), int(ksize[1]), int(ksize[2]),
        int(dilation[0]), int(dilation[1]), int(dilation[2]),
        table.data_ptr(), int(slots), int(key_bits),
        _ptr(out["neighbor_map"]), _ptr(out["gray_code"]), _ptr(out["binary_code"]),
        out["block_offsets"].data_ptr(), meta.data_ptr(),
        meta.data_ptr() + 4 * (V + 2), _stream(dev))
    _cabi.check(rc, "fgb_subm_build_neighbor_map")
    # order check + column index, table clear, insert, hash lookup, column lookup, block scan (with the prefix)
    _count(6)
    return out


def sparse_out_grid(shape, ksize, stride, padding, dilation) -> Tuple[int, int, int]:
    import ctypes
    _, _, W, H, D = [int(s) for s in shape]
    wo, ho, do = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    rc = _cabi.lib().fgb_sparse_out_grid(W, H, D, *[int(v) for v in (*ksize, *stride, *padding, *dilation)],
                                         ctypes.byref(wo), ctypes.byref(ho), ctypes.byref(do))
    _cabi.check(rc, "fgb_sparse_out_grid")
    return wo.value, ho.value, do.value


def sparse_out_coords(coords: torch.Tensor, shape, ksize, stride, padding, dilation, ratio: float, mode: int) -> torch.Tensor:
    """Output coordinates [L,4] int32 of a generic sparse conv, sorted by the
    serialisation key of ``mode`` (0 bxyz, 1 Morton, 2 Hilbert).  One host read
    (the count) between the two library calls."""
    _require_cuda(coords, "coords")
    lib = _cabi.lib()
    dev = coords.device
    n = coords.shape[0]
    B, _, W, H, D = [int(s) for s in shape]
    geom = [int(v) for v in (*ksize, *stride, *padding, *dilation)]
    Wo, Ho, Do = sparse_out_grid(shape, ksize, stride, padding, dilation)
    if n == 0 or min(Wo, Ho, Do) <= 0:
        return torch.empty((0, 4), dtype=torch.int32, device=dev)
    V = geom[0] * geom[1] * geom[2]
    vol = B * Wo * Ho * Do
    key_bits = 32 if vol < 2 ** 32 - 1 else 64
    # as many slots as the reference gives its set (ratio * V / prod(stride) per input voxel), but never fewer
    # than the candidates that can be distinct
    import math
    per_axis = [-(-k // (s // math.gcd(s, d))) for k, s, d in zip(geom[0:3], geom[3:6], geom[9:12])]
    distinct = min(n * per_axis[0] * per_axis[1] * per_axis[2], vol)
    slots = max(int(ratio * V / (geom[3] * geom[4] * geom[5]) * n), int(1.1 * distinct) + 16)
    words = torch.empty((2 * slots * (key_bits // 8) + 7) // 8 + 1, dtype=torch.int64, device=dev)
    set_mem, keys = words, words[(slots * (key_bits // 8) + 7) // 8:]
    count = torch.zeros(2, dtype=torch.int32, device=dev)  # [count, status]
    rc = lib.fgb_sparse_out_coords_collect(_ptr(coords), n, W, H, D, *geom, set_mem.data_ptr(), slots, key_bits, keys.data_ptr(),
                                           count.data_ptr(), count.data_ptr() + 4, _stream(dev))
    _cabi.check(rc, "fgb_sparse_out_coords_collect")
    _count(1)
    host = count.cpu()
    raise_for_status(int(host[1]))
    L = int(host[0])
    out = torch.empty((L, 4), dtype=torch.int32, device=dev)
    if L == 0:
        return out
    nbytes = _cabi.check_size(lib.fgb_sparse_out_coords_workspace_bytes(L, key_bits, int(mode)), "fgb_sparse_out_coords_workspace_bytes")
    ws = workspace(dev, "out_coords", nbytes)
    coord_bits = max((max(W, H, D) - 1).bit_length(), 1)
    rc = lib.fgb_sparse_out_coords_finalize(keys.data_ptr(), L, key_bits, int(mode), coord_bits, B, W, H, D, *geom, ws.data_ptr(),
                                            ws.numel() * 8, out.data_ptr(), _stream(dev))
    _cabi.check(rc, "fgb_sparse_out_coords_finalize")
    _count(2 if mode else 1)
    return out


def sparse_build_neighbor_map(coords: torch.Tensor, out_coords: torch.Tensor, shape, ksize, stride, padding, dilation,
                              table: torch.Tensor, key_bits: int, slots: int, include_bwd: bool) -> Dict[str, torch.Tensor]:
    """Forward map [L,V] (+ backward map [M,V]) of a generic sparse conv with the
    same side products as ``subm_build_neighbor_map`` (they describe the forward map)."""
    _require_cuda(coords, "coords")
    lib = _cabi.lib()
    dev = coords.device
    m, n = coords.shape[0], out_coords.shape[0]
    _, _, W, H, D = [int(s) for s in shape]
    geom = [int(v) for v in (*ksize, *stride, *padding, *dilation)]
    V = geom[0] * geom[1] * geom[2]
    nblk = _cabi.check_size(lib.fgb_map_num_blocks(n), "fgb_map_num_blocks")
    meta = torch.zeros(V + 2, dtype=torch.uint32, device=dev)
    out = {
        "neighbor_map": torch.empty((n, V), dtype=torch.uint32, device=dev),
        "neighbor_map_bwd": torch.empty((m, V), dtype=torch.uint32, device=dev) if include_bwd else None,
        "gray_code": torch.empty(n, dtype=torch.int32, device=dev),
        "binary_code": torch.empty(n, dtype=torch.int32, device=dev),
        "block_offsets": torch.empty(max(V * nblk, 1), dtype=torch.uint32, device=dev),
        "valid_signal_seg": meta[:V + 1],
        "meta": meta,
    }
    rc = lib.fgb_sparse_build_neighbor_map(
        _ptr(coords), m, _ptr(out_coords), n, W, H, D, *geom, table.data_ptr(), int(slots), int(key_bits),
        _ptr(out["neighbor_map"]), _ptr(out["neighbor_map_bwd"]), _ptr(out["gray_code"]), _ptr(out["binary_code"]),
        out["block_offsets"].data_ptr(), meta.data_ptr(), meta.data_ptr() + 4 * (V + 1), _stream(dev))
    _cabi.check(rc, "fgb_sparse_build_neighbor_map")
    _count(4)
    return out


def gray_code_from_map(neighbor_map: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """(gray_code, binary_code), int32 [rows] each, of an existing map."""
    dev = neighbor_map.device
    n, V = neighbor_map.shape
    gray = torch.empty(n, dtype=torch.int32, device=dev)
    binary = torch.empty(n, dtype=torch.int32, device=dev)
    rc = _cabi.lib().fgb_pp_gray_code(_ptr(neighbor_map), n, V, _ptr(gray), _ptr(binary), _stream(dev))
    _cabi.check(rc, "fgb_pp_gray_code")
    _count(1)
    return gray, binary


_meta_host: Dict[tuple, tuple] = {}


def fetch_meta_async(meta: torch.Tensor):
    """Queues the device-to-host copy of a build's ``meta`` words into a pinned
    buffer that is reused between builds (the previous build's read has always
    completed: every build waits for its own copy) and returns ``(host, event)``;
    ``event.synchronize()`` makes ``host`` valid."""
    dev = meta.device
    key = (dev.index, int(meta.numel()))
    entry = _meta_host.get(key)
    if entry is None:
        host = torch.empty(meta.shape, dtype=meta.dtype, pin_memory=True)
        # the numpy view shares the pinned memory: scalar reads without building tensors
        entry = _meta_host[key] = (host, torch.cuda.Event(), host.view(torch.int32).numpy().view("uint32"))
    host, event, host_np = entry
    _cabi.check(_cabi.lib().fgb_fetch_words_async(host.data_ptr(), meta.data_ptr(), meta.numel() * meta.element_size(), _stream(dev)),
                "fgb_fetch_words_async")
    if dev.index is None or dev.index == torch.cuda.current_device():
        event.record()  # torch's current stream of the current device, without building a Stream object
    else:
        event.record(torch.cuda.current_stream(dev))
    return host_np, event


def raise_for_status(code: int) -> None:
    if code != 0:
        what = {_cabi.S_TABLE_FULL: "hash table full (raise the hashmap ratio)",
                _cabi.S_WAIT_TIMEOUT: "a bounded barrier wait ran out inside a kernel"}.get(code, f"code {code}")
        raise RuntimeError(f"flexgemm_b200 device-side error: {what}")


def sorted_idx_from_binary(binary_code: torch.Tensor, key_bits: int) -> torch.Tensor:
    """int64 stable argsort of the binary code (the library's own radix sort over ``key_bits`` bits)."""
    lib = _cabi.lib()
    dev = binary_code.device
    n = binary_code.shape[0]
    out = torch.empty(n, dtype=torch.int64, device=dev)
    if n == 0:
        return out
    nbytes = _cabi.check_size(lib.fgb_pp_sorted_idx_workspace_bytes(n), "fgb_pp_sorted_idx_workspace_bytes")
    ws = workspace(dev, "sort", nbytes)
    rc = lib.fgb_pp_sorted_idx(binary_code.data_ptr(), n, int(key_bits), out.data_ptr(), ws.data_ptr(), ws.numel() * 8,
                               status_word(dev).data_ptr(), _stream(dev))
    _cabi.check(rc, "fgb_pp_sorted_idx")
    _count(1 + (int(key_bits) + 8) // 9)   # digit histogram + one kernel per 9-bit digit
    return out


def valid_signal(neighbor_map: torch.Tensor, gray_code: torch.Tensor, block_offsets: torch.Tensor,
                 valid_signal_seg: torch.Tensor, num_pairs: int,
                 order_flag: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """(valid_signal_i, valid_signal_o), uint32 [num_pairs] each.  ``order_flag``: the submanifold build's word that is
    0 when the rows were in key order (the lists then follow from the masks, the map is not read)."""
    lib = _cabi.lib()
    dev = neighbor_map.device
    n, V = neighbor_map.shape
    vs_i = torch.empty(num_pairs, dtype=torch.uint32, device=dev)
    vs_o = torch.empty(num_pairs, dtype=torch.uint32, device=dev)
    rc = lib.fgb_pp_valid_signal(_ptr(neighbor_map), _ptr(gray_code), n, V, block_offsets.data_ptr(),
                                 valid_signal_seg.data_ptr(), _ptr(vs_i), _ptr(vs_o), _ptr(order_flag), _stream(dev))
    _cabi.check(rc, "fgb_pp_valid_signal")
    _count(1)
    return vs_i, vs_o


def tile_masks(gray_code: torch.Tensor, sorted_idx: torch.Tensor, block: int) -> torch.Tensor:
    lib = _cabi.lib()
    dev = gray_code.device
    n = gray_code.shape[0]
    nblk = (n + block - 1) // block
    out = torch.empty(nblk, dtype=torch.uint32, device=dev)
    rc = lib.fgb_pp_tile_masks(_ptr(gray_code), _ptr(sorted_idx), n, int(block), _ptr(out), _stream(dev))
    _cabi.check(rc, "fgb_pp_tile_masks")
    _count(1)
    return out


def block_schedule(masks: torch.Tensor) -> torch.Tensor:
    """256-row blocks in descending order of work, for the persistent conv kernels."""
    dev = masks.device
    nt = masks.shape[0]
    out = torch.empty(max((nt + 1) // 2, 1), dtype=torch.uint32, device=dev)
    rc = _cabi.lib().fgb_conv_block_schedule(_ptr(masks), nt, out.data_ptr(), _stream(dev))
    _cabi.check(rc, "fgb_conv_block_schedule")
    _count(1)
    return out


def valid_kernel(masks: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """List form of the tile masks: (valid_kernel int32 [sum popcount],
    valid_kernel_seg int32 [nblk+1]).  Synchronises once to size the list, as
    the reference does (migemm_neighmap_pp.cu:356)."""
    lib = _cabi.lib()
    dev = masks.device
    nblk = masks.shape[0]
    seg = torch.empty(nblk + 1, dtype=torch.int32, device=dev)
    vk = torch.empty(max(nblk * 32, 1), dtype=torch.int32, device=dev)
    rc = lib.fgb_pp_valid_kernel(_ptr(masks), nblk, vk.data_ptr(), seg.data_ptr(), _stream(dev))
    _cabi.check(rc, "fgb_pp_valid_kernel")
    _count(1)
    total = int(seg[-1].item())
    return vk[:total].clone(), seg


# --------------------------------------------------------------------------
# conv kernels
# --------------------------------------------------------------------------
def conv_tile_rows() -> int:
    return int(_cabi.lib().fgb_conv_tile_rows())


def set_wgrad_row_bands(bands: int) -> int:
    """Fix the number of row bands of the wgrad pair-list walk (0 = automatic); returns the previous setting."""
    prev = _cabi.lib().fgb_wgrad_set_row_bands(int(bands))
    if prev < 0:
        _cabi.check(prev, "fgb_wgrad_set_row_bands")
    return prev


def set_conv_splitk(splits: int) -> int:
    """Split-K of fprop / dgrad: 0 = automatic (small launches only), 1 = off, k = k shares; returns the previous setting."""
    prev = _cabi.lib().fgb_conv_set_splitk(int(splits))
    if prev < 0:
        _cabi.check(prev, "fgb_conv_set_splitk")
    return prev


MB_TMA, MB_GATHER, MB_MMA, MB_COUPLED, MB_GATHER4, MB_PAIR, MB_LEAN = 1, 2, 4, 8, 16, 32, 64
MB_M64, MB_STORE, MB_STORE_BULK128, MB_STORE_BULK512 = 128, 256, 512, 1024


def microbench_pipeline(mode: int, rows: torch.Tensor, dense: torch.Tensor, iters: int = 2000, stages_a: int = 3, stages_b: int = 3,
                        issue_delay: int = 0):
    """One launch of the pipeline microbenchmark (``fgb_microbench_pipeline``): the operand streams and the MMAs of an
    fprop stage on every SM.  ``rows`` [n, row_bytes / 2] 16-bit, ``dense`` any contiguous buffer.  Returns
    ``(ms, counters)``; counters = the MMA lane's wait cycles / waits for the dense and the gathered operand and the
    total cycles of its loop (CTA 0).  ``issue_delay``: cycles the MMA lane idles before each stage's MMAs."""
    import ctypes
    assert rows.is_cuda and rows.is_contiguous() and rows.element_size() == 2 and dense.is_cuda and dense.is_contiguous()
    ms = ctypes.c_float(0.0)
    counters = (ctypes.c_uint64 * 8)()
    status = status_word(rows.device)
    rc = _cabi.lib().fgb_microbench_pipeline(int(mode), int(stages_a), int(stages_b), int(iters), int(issue_delay), rows.data_ptr(), rows.shape[0],
                                             rows.shape[1] * 2, dense.data_ptr(), dense.numel() * dense.element_size(),
                                             ctypes.byref(ms), counters, status.data_ptr(), _stream(rows.device))
    _count(1)
    _cabi.check(rc, "fgb_microbench_pipeline")
    check_status(rows.device)
    return float(ms.value), [int(c) for c in counters]


def set_conv_dgrad_relayout(on: bool) -> bool:
    """Force dgrad onto the re-laid-out copy of the weight (the path of the 32-bit types) for every type; returns the
    previous setting.  The default reads 16-bit weights as stored."""
    prev = _cabi.lib().fgb_conv_set_dgrad_relayout(1 if on else 0)
    if prev < 0:
        _cabi.check(prev, "fgb_conv_set_dgrad_relayout")
    return bool(prev)


def set_conv_cta_limit(max_ctas: int) -> int:
    """Cap the CTAs (SMs) of the persistent fprop / dgrad kernels launched from now
    on (0 = no cap); returns the previous cap."""
    prev = _cabi.lib().fgb_conv_set_cta_limit(int(max_ctas))
    if prev < 0:
        _cabi.check(prev, "fgb_conv_set_cta_limit")
    return prev


def sm_count(device) -> int:
    return torch.cuda.get_device_properties(device).multi_processor_count


def _channel_multiple(dtype: torch.dtype) -> int:
    """Channel counts the kernels take directly: rows must be whole 16-byte pieces."""
    return 16 // torch.empty(0, dtype=dtype).element_size()


def _round_up(c: int, m: int) -> int:
    return (c + m - 1) // m * m


def _pad_last(t: Optional[torch.Tensor], width: int) -> Optional[torch.Tensor]:
    """``t`` with its last dimension zero-padded to ``width`` (unchanged when it already has it)."""
    if t is None or t.shape[-1] == width:
        return t
    out = t.new_zeros(*t.shape[:-1], width)
    out[..., :t.shape[-1]] = t
    return out


def _pad_weight(weight_cvc: torch.Tensor, co_p: int, ci_p: int) -> torch.Tensor:
    Co, V, Ci = weight_cvc.shape
    if (Co, Ci) == (co_p, ci_p):
        return weight_cvc
    out = weight_cvc.new_zeros(co_p, V, ci_p)
    out[:Co, :, :Ci] = weight_cvc
    return out


def conv_fprop(feats, weight_cvc, bias, neighbor_map, sorted_idx, masks, order=None) -> torch.Tensor:
    """feats [N_in,Ci], weight_cvc [Co,V,Ci], neighbor_map [N_out,V] -> out [N_out,Co]
    (N_in = N_out for a submanifold conv).  Channel counts that do not make the
    rows whole 16-byte pieces (a first layer with Ci = 1, 3, 6 ...) are zero-padded
    to the next multiple and the result is sliced back."""
    lib = _cabi.lib()
    dev = feats.device
    m = _channel_multiple(feats.dtype)
    if feats.shape[1] % m or weight_cvc.shape[0] % m:
        Co = weight_cvc.shape[0]
        ci_p, co_p = _round_up(feats.shape[1], m), _round_up(Co, m)
        out = conv_fprop(_pad_last(feats, ci_p), _pad_weight(weight_cvc, co_p, ci_p), _pad_last(bias, co_p), neighbor_map, sorted_idx,
                         masks, order)
        return out[:, :Co].contiguous()
    poll_status(dev)
    n_in, Ci = feats.shape
    n = neighbor_map.shape[0]
    Co, V, _ = weight_cvc.shape
    code = dtype_code(feats.dtype)
    out = torch.empty((n, Co), dtype=feats.dtype, device=dev)
    nbytes = _cabi.check_size(lib.fgb_sparse_conv_workspace_bytes(0, n, n_in, Ci, Co, V, code, 1), "fgb_sparse_conv_workspace_bytes")
    ws = workspace(dev, "fprop", nbytes)
    if n_in == n:
        rc = lib.fgb_subm_conv_fprop(_ptr(feats), weight_cvc.data_ptr(), _ptr(bias), _ptr(neighbor_map), _ptr(sorted_idx),
                                     _ptr(masks), _ptr(order), _ptr(out), n, Ci, Co, V, code, ws.data_ptr(), ws.numel() * 8,
                                     status_word(dev).data_ptr(), _stream(dev))
        _cabi.check(rc, "fgb_subm_conv_fprop")
    else:
        rc = lib.fgb_sparse_conv_fprop(_ptr(feats), weight_cvc.data_ptr(), _ptr(bias), _ptr(neighbor_map), _ptr(sorted_idx),
                                       _ptr(masks), _ptr(order), _ptr(out), n, n_in, Ci, Co, V, code, ws.data_ptr(),
                                       ws.numel() * 8, status_word(dev).data_ptr(), _stream(dev))
        _cabi.check(rc, "fgb_sparse_conv_fprop")
    _count(1)   # (+ the slab reduction of a split launch, not counted)
    return out


ACTIVATIONS = {None: 0, "none": 0, "silu": 1}  # FGB_ACT_*


def conv_fprop_fused(feats, weight_cvc, bias, neighbor_map, sorted_idx, masks, order=None, activation=None, residual=None,
                     keep_preact: bool = False):
    """Submanifold fprop with ``activation`` (None or "silu") and ``+ residual``
    [N,Co] done in the kernel's epilogue.  Returns (out, preact): preact is the
    conv result before the activation when ``keep_preact`` (else None)."""
    if activation not in ACTIVATIONS:
        raise ValueError(f"Unsupported activation {activation!r}")
    lib = _cabi.lib()
    dev = feats.device
    poll_status(dev)
    n, Ci = feats.shape
    assert neighbor_map.shape[0] == n, "the fused epilogue serves the submanifold conv (one output row per input row)"
    Co, V, _ = weight_cvc.shape
    if residual is not None:
        assert residual.shape == (n, Co) and residual.dtype == feats.dtype and residual.is_contiguous(), "residual must be [N, Co], contiguous, of the feature dtype"
    code = dtype_code(feats.dtype)
    out = torch.empty((n, Co), dtype=feats.dtype, device=dev)
    preact = torch.empty_like(out) if keep_preact else None
    nbytes = _cabi.check_size(lib.fgb_sparse_conv_workspace_bytes(0, n, n, Ci, Co, V, code, 1), "fgb_sparse_conv_workspace_bytes")
    ws = workspace(dev, "fprop", nbytes)
    rc = lib.fgb_subm_conv_fprop_fused(_ptr(feats), weight_cvc.data_ptr(), _ptr(bias), _ptr(residual), _ptr(neighbor_map),
                                       _ptr(sorted_idx), _ptr(masks), _ptr(order), _ptr(out), _ptr(preact), n, Ci, Co, V, code,
                                       ACTIVATIONS[activation], ws.data_ptr(), ws.numel() * 8, status_word(dev).data_ptr(),
                                       _stream(dev))
    _cabi.check(rc, "fgb_subm_conv_fprop_fused")
    _count(1)
    return out, preact


def conv_dgrad(grad_out, weight_cvc, neighbor_map, sorted_idx, masks, order=None, mirror: bool = True) -> torch.Tensor:
    """grad_out [N_out,Co], weight_cvc [Co,V,Ci] -> grad_feats [N_in,Ci].

    ``mirror=True``: ``neighbor_map`` is the forward map of a submanifold conv
    (N_in = N_out; offset v pairs with weight slot V-1-v).  ``mirror=False``:
    it is the backward map [N_in, V] of a generic sparse conv (slot v)."""
    lib = _cabi.lib()
    dev = grad_out.device
    m = _channel_multiple(grad_out.dtype)
    if grad_out.shape[1] % m or weight_cvc.shape[2] % m:
        Ci = weight_cvc.shape[2]
        ci_p, co_p = _round_up(Ci, m), _round_up(grad_out.shape[1], m)
        out = conv_dgrad(_pad_last(grad_out, co_p), _pad_weight(weight_cvc, co_p, ci_p), neighbor_map, sorted_idx, masks, order, mirror)
        return out[:, :Ci].contiguous()
    poll_status(dev)
    n_out, Co = grad_out.shape
    n = neighbor_map.shape[0]
    _, V, Ci = weight_cvc.shape
    code = dtype_code(grad_out.dtype)
    out = torch.empty((n, Ci), dtype=grad_out.dtype, device=dev)
    nbytes = _cabi.check_size(lib.fgb_sparse_conv_workspace_bytes(1, n_out, n, Ci, Co, V, code, 1), "fgb_sparse_conv_workspace_bytes")
    ws = workspace(dev, "dgrad", nbytes)
    if mirror:
        assert n == n_out, "a mirrored (submanifold) dgrad needs as many map rows as grad_out rows"
        rc = lib.fgb_subm_conv_dgrad(_ptr(grad_out), weight_cvc.data_ptr(), _ptr(neighbor_map), _ptr(sorted_idx), _ptr(masks),
                                     _ptr(order), _ptr(out), n, Ci, Co, V, code, ws.data_ptr(), ws.numel() * 8,
                                     status_word(dev).data_ptr(), _stream(dev))
        _cabi.check(rc, "fgb_subm_conv_dgrad")
    else:
        rc = lib.fgb_sparse_conv_dgrad(_ptr(grad_out), weight_cvc.data_ptr(), _ptr(neighbor_map), _ptr(sorted_idx), _ptr(masks),
                                       _ptr(order), _ptr(out), n, n_out, Ci, Co, V, code, ws.data_ptr(), ws.numel() * 8,
                                       status_word(dev).data_ptr(), _stream(dev))
        _cabi.check(rc, "fgb_sparse_conv_dgrad")
    _count(2)
    return out


def conv_wgrad(grad_out, feats, vs_i, vs_o, vs_seg, splitk: Optional[int] = None, want_f32: bool = False,
               want_dtype: bool = True, block_offsets: Optional[torch.Tensor] = None, out_f32: Optional[torch.Tensor] = None):
    """-> (grad_weight [Co,V,Ci] in the feature dtype or None, fp32 copy or None).
    ``block_offsets`` (the build's per-(offset, 256-row block) pair offsets) lets
    the kernel walk all pair lists in row bands that the offsets share in L2.
    ``out_f32`` (fp32, Co*V*Ci elements, contiguous) receives the fp32 copy in
    place -- e.g. a slice of the buffer a multi-GPU caller all-reduces."""
    lib = _cabi.lib()
    dev = feats.device
    n_in, Ci = feats.shape
    n_out, Co = grad_out.shape
    m = _channel_multiple(feats.dtype)
    if (Ci % m or Co % m) and out_f32 is not None:
        gw, gw32 = conv_wgrad(grad_out, feats, vs_i, vs_o, vs_seg, splitk, True, want_dtype, block_offsets)
        out_f32.view(gw32.shape).copy_(gw32)
        return gw, out_f32.view(gw32.shape)
    if Ci % m or Co % m:
        gw, gw32 = conv_wgrad(_pad_last(grad_out, _round_up(Co, m)), _pad_last(feats, _round_up(Ci, m)), vs_i, vs_o, vs_seg, splitk,
                              want_f32, want_dtype, block_offsets)
        return (gw[:Co, :, :Ci].contiguous() if gw is not None else None,
                gw32[:Co, :, :Ci].contiguous() if gw32 is not None else None)
    poll_status(dev)
    V = vs_seg.shape[0] - 1
    code = dtype_code(feats.dtype)
    if splitk is None:
        splitk = lib.fgb_wgrad_default_splitk(int(vs_i.shape[0]), Ci, Co, V, code)
        if splitk < 1:
            _cabi.check(splitk, "fgb_wgrad_default_splitk")
    gw = torch.empty((Co, V, Ci), dtype=feats.dtype, device=dev) if want_dtype else None
    if out_f32 is not None:
        assert out_f32.dtype == torch.float32 and out_f32.numel() == Co * V * Ci and out_f32.is_contiguous()
        gw32 = out_f32.view(Co, V, Ci)
    else:
        gw32 = torch.empty((Co, V, Ci), dtype=torch.float32, device=dev) if want_f32 else None
    nbytes = _cabi.check_size(lib.fgb_sparse_conv_workspace_bytes(2, n_out, n_in, Ci, Co, V, code, splitk),
                              "fgb_sparse_conv_workspace_bytes")
    ws = workspace(dev, "wgrad", nbytes)
    if n_in == n_out:
        rc = lib.fgb_subm_conv_wgrad(_ptr(grad_out), _ptr(feats), _ptr(vs_i), _ptr(vs_o), vs_seg.data_ptr(), _ptr(block_offsets), _ptr(gw), _ptr(gw32),
                                     n_out, int(vs_i.shape[0]), Ci, Co, V, code, int(splitk), ws.data_ptr(), ws.numel() * 8,
                                     status_word(dev).data_ptr(), _stream(dev))
        _cabi.check(rc, "fgb_subm_conv_wgrad")
    else:
        rc = lib.fgb_sparse_conv_wgrad(_ptr(grad_out), _ptr(feats), _ptr(vs_i), _ptr(vs_o), vs_seg.data_ptr(), _ptr(block_offsets), _ptr(gw),
                                       _ptr(gw32), n_out, n_in, int(vs_i.shape[0]), Ci, Co, V, code, int(splitk), ws.data_ptr(),
                                       ws.numel() * 8, status_word(dev).data_ptr(), _stream(dev))
        _cabi.check(rc, "fgb_sparse_conv_wgrad")
    _count(2)
    return gw, gw32


def bias_grad(grad_out, want_f32: bool = False, want_dtype: bool = True, out_f32: Optional[torch.Tensor] = None):
    """-> (grad_bias [Co] in the feature dtype or None, fp32 copy or None); ``out_f32`` receives the fp32 copy in place."""
    lib = _cabi.lib()
    dev = grad_out.device
    n, Co = grad_out.shape
    code = dtype_code(grad_out.dtype)
    gb = torch.empty(Co, dtype=grad_out.dtype, device=dev) if want_dtype else None
    if out_f32 is not None:
        assert out_f32.dtype == torch.float32 and out_f32.shape == (Co,) and out_f32.is_contiguous()
        gb32 = out_f32
    else:
        gb32 = torch.empty(Co, dtype=torch.float32, device=dev) if want_f32 else None
    nbytes = _cabi.check_size(lib.fgb_bias_grad_workspace_bytes(Co), "fgb_bias_grad_workspace_bytes")
    ws = workspace(dev, "bias", nbytes)
    rc = lib.fgb_subm_conv_bias_grad(_ptr(grad_out), _ptr(gb), _ptr(gb32), n, Co, code, ws.data_ptr(), ws.numel() * 8, _stream(dev))
    _cabi.check(rc, "fgb_subm_conv_bias_grad")
    _count(2)
    return gb, gb32


_side_streams: Dict[int, "torch.cuda.Stream"] = {}


def bias_grad_overlapped(grad_out, want_f32: bool = False, want_dtype: bool = True, out_f32: Optional[torch.Tensor] = None):
    """Starts the bias gradient on a side stream so that it runs in the shadow of
    the persistent conv kernels (which hold one CTA per SM but leave room for the
    small reduction CTAs), and returns ``(grad_bias, grad_bias_f32, join)``: call
    ``join()`` on the launching stream after the other backward kernels have been
    queued and before the gradient is used."""
    dev = grad_out.device
    cur = torch.cuda.current_stream(dev)
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    side = _side_streams.get(idx)
    if side is None:
        side = _side_streams[idx] = torch.cuda.Stream(device=dev)
    side.wait_stream(cur)                  # grad_out is ready once the launching stream gets here
    with torch.cuda.stream(side):
        gb, gb32 = bias_grad(grad_out, want_f32=want_f32, want_dtype=want_dtype, out_f32=out_f32)
    grad_out.record_stream(side)
    if out_f32 is not None:
        out_f32.record_stream(side)

    def join():
        cur.wait_stream(side)
        for t in (gb, gb32):
            if t is not None:
                t.record_stream(cur)

    return gb, gb32, join


def cast_from_f32(src: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    out = torch.empty(src.shape, dtype=dtype, device=src.device)
    code = _DTYPES.get(dtype, _cabi.F32_TF32)
    rc = _cabi.lib().fgb_cast_from_f32(_ptr(src), _ptr(out), src.numel(), code, _stream(src.device))
    _cabi.check(rc, "fgb_cast_from_f32")
    _count(1)
    return out


# --------------------------------------------------------------------------
# generic table use and grid sample
# --------------------------------------------------------------------------
def table_insert_3d_idx_as_val(table: torch.Tensor, key_bits: int, slots: int, coords: torch.Tensor, W: int, H: int, D: int) -> torch.Tensor:
    """The library's packed table: clears ``table`` and inserts ``coords[i] -> i``; returns this call's device status word."""
    _require_cuda(coords, "coords")
    dev = coords.device
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    rc = _cabi.lib().fgb_hash_insert_3d_idx_as_val(_ptr(coords), coords.shape[0], int(W), int(H), int(D), table.data_ptr(), int(slots),
                                                   int(key_bits), status.data_ptr(), _stream(dev))
    _cabi.check(rc, "fgb_hash_insert_3d_idx_as_val")
    _count(2)
    return status


def table_lookup_3d(table: torch.Tensor, key_bits: int, slots: int, query_coords: torch.Tensor, W: int, H: int, D: int) -> torch.Tensor:
    """The library's packed table: uint32 [M], row stored for each (b, x, y, z) query row, 0xffffffff where absent."""
    dev = query_coords.device
    out = torch.empty(query_coords.shape[0], dtype=torch.uint32, device=dev)
    rc = _cabi.lib().fgb_hash_lookup_3d(_ptr(query_coords), query_coords.shape[0], int(W), int(H), int(D), table.data_ptr(), int(slots),
                                        int(key_bits), _ptr(out), _stream(dev))
    _cabi.check(rc, "fgb_hash_lookup_3d")
    _count(1)
    return out


# The generic hash map in the reference's own layout and call shapes
# (flex_gemm/kernels/cuda/hash/hash.cu; bound in ext.cpp:12-16): a key tensor
# (uint32 / uint64, empty = all ones) and a value tensor (uint32 / uint64).
_BITS = {torch.uint32: 32, torch.uint64: 64}


def _hashmap_args(hashmap_keys: torch.Tensor, hashmap_values: torch.Tensor):
    _require_cuda(hashmap_keys, "hashmap_keys")
    if hashmap_keys.dtype not in _BITS or hashmap_values.dtype not in _BITS:
        raise RuntimeError("Unsupported data type")       # the reference's TORCH_CHECK message
    if hashmap_keys.shape != hashmap_values.shape or hashmap_keys.dim() != 1:
        raise RuntimeError("hashmap_keys and hashmap_values must be 1-D tensors of the same length")
    return hashmap_keys.shape[0], _BITS[hashmap_keys.dtype], _BITS[hashmap_values.dtype]


def _hashmap_status(dev, status: torch.Tensor) -> None:
    raise_for_status(int(status.item()))


def hashmap_insert(hashmap_keys: torch.Tensor, hashmap_values: torch.Tensor, keys: torch.Tensor, values: torch.Tensor) -> None:
    """Insert ``keys[i] -> values[i]`` (hash.cu:60-92).  Synchronises to report a full table."""
    slots, kb, vb = _hashmap_args(hashmap_keys, hashmap_values)
    if keys.dtype != hashmap_keys.dtype:
        raise RuntimeError(f"Keys must be {str(hashmap_keys.dtype).split('.')[-1]}")
    if values.dtype != hashmap_values.dtype:
        raise RuntimeError(f"Values must be {str(hashmap_values.dtype).split('.')[-1]}")
    dev = hashmap_keys.device
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    keys, values = keys.contiguous(), values.contiguous()
    rc = _cabi.lib().fgb_hashmap_insert(hashmap_keys.data_ptr(), hashmap_values.data_ptr(), slots, kb, vb, _ptr(keys), _ptr(values),
                                        keys.shape[0], status.data_ptr(), _stream(dev))
    _cabi.check(rc, "fgb_hashmap_insert")
    _count(1)
    _hashmap_status(dev, status)


def hashmap_lookup(hashmap_keys: torch.Tensor, hashmap_values: torch.Tensor, keys: torch.Tensor) -> torch.Tensor:
    """Values of ``keys`` (all ones where absent), in the value dtype (hash.cu:139-175)."""
    slots, kb, vb = _hashmap_args(hashmap_keys, hashmap_values)
    if keys.dtype != hashmap_keys.dtype:
        raise RuntimeError(f"Keys must be {str(hashmap_keys.dtype).split('.')[-1]}")
    dev = hashmap_keys.device
    keys = keys.contiguous()
    out = torch.empty(keys.shape[0], dtype=hashmap_values.dtype, device=dev)
    rc = _cabi.lib().fgb_hashmap_lookup(hashmap_keys.data_ptr(), hashmap_values.data_ptr(), slots, kb, vb, _ptr(keys), keys.shape[0],
                                        _ptr(out), _stream(dev))
    _cabi.check(rc, "fgb_hashmap_lookup")
    _count(1)
    return out


def hashmap_insert_3d(hashmap_keys: torch.Tensor, hashmap_values: torch.Tensor, coords: torch.Tensor, values: torch.Tensor,
                      W: int, H: int, D: int) -> None:
    """Insert ``coords[i] (b, x, y, z) -> values[i]`` under the flat index (hash.cu:237-270)."""
    slots, kb, vb = _hashmap_args(hashmap_keys, hashmap_values)
    if coords.dtype != torch.int32:
        raise RuntimeError("Coords must be int32")
    if values.dtype != hashmap_values.dtype:
        raise RuntimeError(f"Values must be {str(hashmap_values.dtype).split('.')[-1]}")
    dev = hashmap_keys.device
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    coords, values = coords.contiguous(), values.contiguous()
    rc = _cabi.lib().fgb_hashmap_insert_3d(hashmap_keys.data_ptr(), hashmap_values.data_ptr(), slots, kb, vb, _ptr(coords), _ptr(values),
                                           coords.shape[0], int(W), int(H), int(D), status.data_ptr(), _stream(dev))
    _cabi.check(rc, "fgb_hashmap_insert_3d")
    _count(1)
    _hashmap_status(dev, status)


def hashmap_insert_3d_idx_as_val(hashmap_keys: torch.Tensor, hashmap_values: torch.Tensor, coords: torch.Tensor,
                                 W: int, H: int, D: int) -> None:
    """Insert ``coords[i] -> i`` (hash.cu:425-449)."""
    slots, kb, vb = _hashmap_args(hashmap_keys, hashmap_values)
    if coords.dtype != torch.int32:
        raise RuntimeError("Coords must be int32")
    dev = hashmap_keys.device
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    coords = coords.contiguous()
    rc = _cabi.lib().fgb_hashmap_insert_3d_idx_as_val(hashmap_keys.data_ptr(), hashmap_values.data_ptr(), slots, kb, vb, _ptr(coords),
                                                      coords.shape[0], int(W), int(H), int(D), status.data_ptr(), _stream(dev))
    _cabi.check(rc, "fgb_hashmap_insert_3d_idx_as_val")
    _count(1)
    _hashmap_status(dev, status)


def hashmap_lookup_3d(hashmap_keys: torch.Tensor, hashmap_values: torch.Tensor, coords: torch.Tensor, W: int, H: int, D: int) -> torch.Tensor:
    """Values stored for the (b, x, y, z) rows of ``coords`` (all ones where absent or outside the grid; hash.cu:336-365)."""
    slots, kb, vb = _hashmap_args(hashmap_keys, hashmap_values)
    if coords.dtype != torch.int32:
        raise RuntimeError("Coords must be int32")
    dev = hashmap_keys.device
    coords = coords.contiguous()
    out = torch.empty(coords.shape[0], dtype=hashmap_values.dtype, device=dev)
    rc = _cabi.lib().fgb_hashmap_lookup_3d(hashmap_keys.data_ptr(), hashmap_values.data_ptr(), slots, kb, vb, _ptr(coords), coords.shape[0],
                                           int(W), int(H), int(D), _ptr(out), _stream(dev))
    _cabi.check(rc, "fgb_hashmap_lookup_3d")
    _count(1)
    return out


def grid_sample_neighbor_map(table: torch.Tensor, key_bits: int, slots: int, query: torch.Tensor, W: int, H: int, D: int,
                             trilinear: bool):
    """``query`` fp32 [B, L, 3] -> neighbor uint32 [B, L] (nearest) or (neighbor [B, L, 8], weight fp32 [B, L, 8])."""
    dev = query.device
    B, L = query.shape[:2]
    if trilinear:
        nb = torch.empty((B, L, 8), dtype=torch.uint32, device=dev)
        w = torch.empty((B, L, 8), dtype=torch.float32, device=dev)
    else:
        nb = torch.empty((B, L), dtype=torch.uint32, device=dev)
        w = None
    rc = _cabi.lib().fgb_grid_sample_neighbor_map(_ptr(query), B, L, int(W), int(H), int(D), table.data_ptr(), int(slots), int(key_bits),
                                                  1 if trilinear else 0, _ptr(nb), _ptr(w), _stream(dev))
    _cabi.check(rc, "fgb_grid_sample_neighbor_map")
    _count(1)
    return (nb, w) if trilinear else nb


def _elem_code(dtype: torch.dtype) -> int:
    if dtype in _DTYPES:
        return _DTYPES[dtype]
    if dtype == torch.float32:
        return _cabi.F32_IEEE
    raise TypeError(f"unsupported feature dtype {dtype}: expected float16, bfloat16 or float32")


def indice_weighted_sum_fwd(feats: torch.Tensor, indices: torch.Tensor, weight: Optional[torch.Tensor]) -> torch.Tensor:
    """feats [N, C], indices uint32 [M, V], weight fp32 [M, V] or None -> [M, C]."""
    dev = feats.device
    M, V = indices.shape
    C = feats.shape[1]
    out = torch.empty((M, C), dtype=feats.dtype, device=dev)
    rc = _cabi.lib().fgb_indice_weighted_sum_fwd(_ptr(feats), _ptr(indices), _ptr(weight), _ptr(out), M, C, V, _elem_code(feats.dtype),
                                                 _stream(dev))
    _cabi.check(rc, "fgb_indice_weighted_sum_fwd")
    _count(1)
    return out


def indice_weighted_sum_bwd(grad_out: torch.Tensor, indices: torch.Tensor, weight: Optional[torch.Tensor], n: int) -> torch.Tensor:
    """grad_out [M, C] -> fp32 [n, C]: the scatter-add of the weighted rows."""
    dev = grad_out.device
    M, V = indices.shape
    C = grad_out.shape[1]
    out = torch.empty((n, C), dtype=torch.float32, device=dev)
    rc = _cabi.lib().fgb_indice_weighted_sum_bwd(_ptr(grad_out), _ptr(indices), _ptr(weight), _ptr(out), M, n, C, V,
                                                 _elem_code(grad_out.dtype), _stream(dev))
    _cabi.check(rc, "fgb_indice_weighted_sum_bwd")
    _count(1)
    return out
