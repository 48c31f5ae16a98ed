"""Benchmark of the submanifold-conv3d hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One step = forward + backward (dgrad, wgrad, bias grad) of one 3x3x3
submanifold convolution on the headline workload: a spherical shell at
RES=256, C=256 -> 256, fp16, one sample per GPU (weak scaling: with N GPUs the
batch holds N samples, one per rank, and the weight/bias gradient is summed
with one NCCL all-reduce per step).  The reported value is useful TFLOP/s,
6 * L * Ci * Co per step with L = number of valid (voxel, offset) pairs.  The
timed region of K steps is repeated (``--repeats``, 5 by default): ``value``
and ``ms_per_step`` are the median repeat, the spread is in ``repeats``.

Printed JSON (one line, rank 0): the metric and, beside it,
* ``roofline``: the slowest of fprop / dgrad / wgrad timed alone against the
  measured dense tensor peak, ``roofline_map_build`` for the neighbour-cache
  build (both the table-free path sorted input takes and the hash-table path),
* ``sustained``: a back-to-back loop of at least one second against the
  sustained tensor peak, with its own clock record,
* ``e2e``: the same metric through the public API with host buffers,
* ``cpu_baseline``: the explicit gather-GEMM-scatter algorithm of the reference,
  restated in oracle/, timed on this host's cores on a bounded slab,
* one GPU only: ``sweep`` (channel / dtype sweep on the RES=128 shell),
  ``residual_stack`` (16 convs at C=512 bf16, elementwise work as torch kernels
  and fused into the conv epilogues) and ``map_build_res1024`` (the cache build at
  a size where HBM matters),
* ``sharded_batch``: the batch of 8 shells at RES=1024 (C=64) dealt to the N
  ranks by voxel count, strong scaling, next to its load-balance bound,
* N > 1: ``phases`` (every phase of a step timed alone, max over ranks) and
  ``allreduce_check`` (the NCCL-reduced gradient against the sum of every rank's
  local gradient recomputed on rank 0).

--impl reference times the CPU algorithm alone, with all host threads.
--workload res1024_batch8 | res1024_map [--unsorted] | residual_stack [--fused] | pipeline_microbench
run one of the side workloads alone (what the ncu captures under profiles/ use).
--quick skips the side workloads of the default run.
"""
import argparse
import json
import os
import statistics
import sys
import time

import torch

_JSON_OUT = sys.stdout


def claim_stdout() -> None:
    """stdout carries the one JSON line and nothing else: libraries that write there from native code (NCCL prints
    its version line on the first communicator) get stderr instead, and the line goes out through a copy of the real
    stdout.  Called once by main()."""
    global _JSON_OUT
    sys.stdout.flush()
    _JSON_OUT = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)


def emit(line: dict) -> None:
    _JSON_OUT.write(json.dumps(line) + "\n")
    _JSON_OUT.flush()


ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "submconv fwd+bwd useful TFLOP/s (C=256 fp16, RES=256); neighbor-map build ms"
RES, CI, CO = 256, 256, 256
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
# dram__bytes_read.sum + dram__bytes_write.sum per launch at the headline workload, copied from an ncu capture; the
# capture is identified by the commit of the kernels it ran (the kernels may have changed since: compare with HEAD)
NCU_DRAM_TRAFFIC = {
    "commit": "e76fbda",
    "bytes": {"fprop": 290.0e6, "dgrad": 288.5e6, "wgrad": 184.9e6},
}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        p["source"] = "measured"
        return p
    p = dict(FALLBACK_PEAKS)
    p["source"] = "fallback"
    return p


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clock, power and throttle reasons of one GPU through NVML from
    a background thread (read-only queries; about one sample per millisecond, so
    that even a 20 ms timed region is covered)."""

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.samples = []
        self.thread = None
        self.stop_flag = False
        self.nvml = None

    def start(self):
        try:
            import threading

            import pynvml
            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            index = int(visible.split(",")[self.gpu]) if visible and visible.split(",")[self.gpu].isdigit() else self.gpu
            handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.nvml = pynvml
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM)

            def loop():
                while not self.stop_flag:
                    try:
                        mhz = pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM)
                        reasons = pynvml.nvmlDeviceGetCurrentClocksEventReasons(handle)
                        watts = pynvml.nvmlDeviceGetPowerUsage(handle) / 1000.0
                        self.samples.append((mhz, reasons, watts))
                    except Exception:
                        pass
                    time.sleep(0.001)

            self.thread = threading.Thread(target=loop, daemon=True)
            self.thread.start()
        except Exception:
            self.thread = None
        return self

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.thread is None:
            return out
        self.stop_flag = True
        self.thread.join(timeout=2)
        if not self.samples:
            return out
        nv = self.nvml
        names = {"hw_slowdown": nv.nvmlClocksEventReasonHwSlowdown, "hw_thermal_slowdown": nv.nvmlClocksEventReasonHwThermalSlowdown,
                 "sw_thermal_slowdown": nv.nvmlClocksEventReasonSwThermalSlowdown, "sw_power_cap": nv.nvmlClocksEventReasonSwPowerCap}
        seen = set()
        for _, reasons, _ in self.samples:
            for name, bit in names.items():
                if reasons & bit:
                    seen.add(name)
        out["sm_mhz"] = statistics.median(m for m, _, _ in self.samples)
        out["sm_max_mhz"] = self.max_mhz
        out["power_w_max"] = max(w for _, _, w in self.samples)
        out["reasons"] = sorted(seen)
        out["samples"] = len(self.samples)
        return out


# --------------------------------------------------------------------------- CPU arm (oracle port of the reference's explicit path)
def cpu_explicit_steps(steps: int, warmup: int, threads: int):
    """Times fwd+bwd of the explicit gather-GEMM-scatter algorithm on a slab of
    the headline workload: the first 1/8 of the output rows (all 27 offsets,
    full channel width), fp32 on the CPU.  Returns (TFLOP/s, ms/step, sample text)."""
    from oracle import submconv_oracle as orc
    torch.set_num_threads(threads)
    coords = orc.shell_coords(RES)
    shape = (1, CI, RES, RES, RES)
    nbr = orc.neighbor_map(coords, shape)
    n = nbr.shape[0]
    ns = n // 8
    g = torch.Generator().manual_seed(2)
    feats = torch.randn(n, CI, generator=g)
    weight = torch.randn(CO, 27, CI, generator=g) / (27 * CI) ** 0.5
    bias = torch.randn(CO, generator=g)
    gout = torch.ones(n, CO)
    sub = torch.from_numpy(nbr[:ns].astype("int64"))
    pairs = int((nbr[:ns] != orc.INVALID).sum())
    w_fwd = weight.reshape(CO, 27 * CI).t().contiguous()
    w_bwd = weight.transpose(0, 1).reshape(27 * CO, CI).contiguous()

    def step():
        col = orc._im2col(feats, sub, 27)                      # gather
        out = torch.addmm(bias, col, w_fwd)                    # fprop rows [0, ns)
        colg = orc._im2col(gout, torch.flip(sub, [1]), 27)
        gin = torch.mm(colg, w_bwd)                            # dgrad rows [0, ns)
        gw = torch.mm(col.t(), gout[:ns])                      # wgrad contribution of the slab
        gb = gout[:ns].sum(0)
        return out, gin, gw, gb

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    flops = 6.0 * pairs * CI * CO
    sample = f"first {ns} of {n} output rows of the RES={RES} C={CI} shell ({pairs} pairs), fp32, {steps} steps"
    return flops / dt / 1e12, dt * 1e3, sample


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    tflops, ms, sample = cpu_explicit_steps(args.steps, args.warmup, threads)
    ref_map = reference_cuda_map_build()
    line = {
        "impl": "reference", "metric": METRIC, "value": tflops, "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"submconv3d k3 fwd+bwd, spherical shell RES={RES}, Ci=Co={CI}, explicit gather-GEMM-scatter on host cores",
                   "sample": sample},
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "reference_cuda_map_build": ref_map,
    }
    emit(line)


def reference_cuda_map_build():
    """The second half of the metric for the reference: its neighbour-cache build (its own hash table, neighbour-map
    and post-processing kernels, compiled from its sources into oracle/_ref by oracle/build_reference_ext.py) on the
    headline shell, on this machine's GPU.  None where the extension or a GPU is missing."""
    try:
        from oracle.build_reference_ext import load_reference_ext, reference_neighbor_cache
        ref = load_reference_ext()
        if ref is None or not torch.cuda.is_available():
            return None
        from oracle import submconv_oracle as orc
        dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
        coords = torch.from_numpy(orc.shell_coords(RES)).to(dev)
        shape = (1, CI, RES, RES, RES)
        for _ in range(3):
            reference_neighbor_cache(ref, coords, shape)
        ms = time_loop(lambda: reference_neighbor_cache(ref, coords, shape), 20)
        return {"ms": ms, "what": "the reference's compiled CUDA functions (init_hashmap + hashmap_build_submanifold_conv_neighbour_map + "
                                  "neighbor_map_post_process_for_masked_implicit_gemm_1) on the RES=256 shell, rows in key order, 20 builds"}
    except Exception as e:  # the CPU arm must not fail for lack of the optional GPU figure
        return {"ms": None, "error": str(e)[:200]}


# --------------------------------------------------------------------------- GPU helpers
def time_loop(fn, iters: int) -> float:
    """Average milliseconds per call, CUDA events on the current stream."""
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters


def map_build_bytes(n: int, pairs: int, ratio: float, key_bytes: int = 4, V: int = 27) -> int:
    """Algorithmic bytes of one neighbour-cache build: table build + lookup + post-processing."""
    slots = int(ratio * n)
    k = key_bytes
    return (16 * n + k * slots + (k + 4) * n) + (16 * n + 13 * n * k + 4 * (pairs - n) // 2 + 4 * V * n) + \
           (4 * V * n + 4 * n + 8 * n + 8 * pairs)


def dist_env():
    return int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))


def time_map_build(coords, shape, iters: int, warmup: int = 3):
    """(ms per build, cache) of the training neighbour cache of ``coords``."""
    from flexgemm_b200.ops.spconv import SubMConv3dFunction as F

    def build():
        return F._compute_neighbor_cache(coords, shape, (3, 3, 3), (1, 1, 1), True)

    cache = None
    for _ in range(warmup):
        cache = build()
    # the host is part of a build (one round trip): the median of three regions keeps a host stall out of the figure
    return statistics.median(time_loop(build, iters) for _ in range(3)), cache


def map_build_report(coords_sorted, shape, peaks, iters: int):
    """Both paths of the cache build on the same voxels: rows in key order (no table) and shuffled (hash table)."""
    from flexgemm_b200.ops import spconv
    out = {}
    n = coords_sorted.shape[0]
    perm = torch.randperm(n, generator=torch.Generator().manual_seed(1)).to(coords_sorted.device)
    for name, c in (("sorted", coords_sorted), ("hash", coords_sorted[perm].contiguous())):
        ms, cache = time_map_build(c, shape, iters)
        pairs = int(cache["valid_signal_i"].shape[0])
        nbytes = map_build_bytes(n, pairs, spconv.HASHMAP_RATIO)
        gbs = nbytes / (ms * 1e-3) / 1e9
        out[name] = {"ms": ms, "gbs": gbs, "frac": gbs / float(peaks["hbm_gbs"]), "algorithmic_bytes": nbytes}
        del cache
    out["n_voxels"], out["peak_gbs"], out["peak_source"] = n, float(peaks["hbm_gbs"]), peaks["source"]
    return out


# --------------------------------------------------------------------------- side workloads (also reachable alone through --workload)
def sweep_report(dev, peaks, iters: int = 8):
    """Channel / dtype sweep on the RES=128 shell: fwd + bwd per point, useful TFLOP/s against the dense tensor
    peak of the type (C >= 256) and gathered bytes per second against HBM (C <= 128, where the gather bounds it)."""
    from flexgemm_b200 import workloads
    from flexgemm_b200.kernels import cuda as K
    from flexgemm_b200.ops.spconv import SubMConv3dFunction as F
    res = 128
    coords = workloads.shell_coords_torch(res, device=dev)
    n = coords.shape[0]
    peak16 = float(peaks["bf16_tflops"])
    points = []
    cache = F._compute_neighbor_cache(coords, torch.Size((1, 64, res, res, res)), (3, 3, 3), (1, 1, 1), True)
    cache.block_order(K.conv_tile_rows())
    pairs = int(cache["valid_signal_i"].shape[0])
    for dtype, name, peak in ((torch.float16, "f16", peak16), (torch.float32, "tf32", peak16 / 2)):
        for c in (64, 128, 256, 512, 1024):
            g = torch.Generator(device=dev).manual_seed(3)
            feats = torch.randn(n, c, generator=g, device=dev).to(dtype)
            gout = torch.randn(n, c, generator=g, device=dev).to(dtype)
            weight = (torch.randn(c, 3, 3, 3, c, generator=g, device=dev) / (27 * c) ** 0.5).to(dtype)
            bias = torch.randn(c, generator=g, device=dev).to(dtype)
            f_req, w_req, b_req = (t.detach().requires_grad_(True) for t in (feats, weight, bias))

            def step():
                F._sparse_submanifold_conv_forward(feats, cache, weight, bias)
                F._sparse_submanifold_conv_backward(gout, f_req, cache, w_req, b_req)

            for _ in range(3):
                step()
            ms = statistics.median(time_loop(step, iters) for _ in range(3))
            tf = 6.0 * pairs * c * c / (ms * 1e-3) / 1e12
            eb = feats.element_size()
            gathered = 4.0 * pairs * c * eb            # fprop + dgrad one gathered operand each, wgrad two
            gbs = gathered / (ms * 1e-3) / 1e9
            points.append({"dtype": name, "C": c, "ms": round(ms, 4), "tflops": round(tf, 1), "frac_tensor": round(tf / peak, 4),
                           "gathered_gbs": round(gbs, 1), "frac_hbm": round(gbs / float(peaks["hbm_gbs"]), 4),
                           "bound": "tensor" if c >= 256 else "gather"})
            del feats, gout, weight, f_req, w_req, step
    K.check_status(dev)
    return {"workload": f"RES=128 shell, N={n} voxels, L={pairs} pairs, k3 fwd+bwd, cache reused",
            "tf32_peak": "half of the measured bf16 peak", "points": points}


def residual_stack_steps(dev, fused: bool, steps: int, warmup: int = 3):
    """Residual stack: 8 blocks [conv, SiLU, conv] + skip on 4 shells at RES=64,
    C=512, bf16, one shared neighbour cache, forward + backward of the mean.
    ``fused``: SiLU and the skip addition run in the conv kernels' epilogue."""
    from flexgemm_b200 import workloads
    from flexgemm_b200.kernels import cuda as K
    from flexgemm_b200.ops import spconv
    from flexgemm_b200.ops.spconv import SubMConv3dFunction as F
    B, res, C, blocks = 4, 64, 512, 8
    dt = torch.bfloat16
    coords = workloads.shell_coords_torch(res, B, [1.0] * B, device=dev)
    shape = torch.Size((B, C, res, res, res))
    g = torch.Generator().manual_seed(5)
    x0 = torch.randn(coords.shape[0], C, generator=g).to(dt).to(dev)
    ws = [(torch.randn(C, 3, 3, 3, C, generator=g) / (27 * C) ** 0.5).to(dt).to(dev).requires_grad_(True) for _ in range(2 * blocks)]
    bs = [torch.zeros(C, dtype=dt, device=dev).requires_grad_(True) for _ in range(2 * blocks)]
    cache = F._compute_neighbor_cache(coords, shape, (3, 3, 3), (1, 1, 1), True)
    pairs = int(cache["valid_signal_i"].shape[0])

    def step():
        h = x0.detach().requires_grad_(True)
        for i in range(blocks):
            if fused:
                y, _ = spconv.sparse_submanifold_conv3d_fused(h, coords, shape, ws[2 * i], bs[2 * i], neighbor_cache=cache, activation="silu")
                h, _ = spconv.sparse_submanifold_conv3d_fused(y, coords, shape, ws[2 * i + 1], bs[2 * i + 1], neighbor_cache=cache, residual=h)
            else:
                y, _ = spconv.sparse_submanifold_conv3d(h, coords, shape, ws[2 * i], bs[2 * i], neighbor_cache=cache)
                y = torch.nn.functional.silu(y)
                y, _ = spconv.sparse_submanifold_conv3d(y, coords, shape, ws[2 * i + 1], bs[2 * i + 1], neighbor_cache=cache)
                h = h + y
        h.float().mean().backward()
        for t in ws + bs:
            t.grad = None

    for _ in range(warmup):
        step()
    K.check_status(dev)
    launches0 = K.launch_count
    ms = time_loop(step, steps)
    launches = K.launch_count - launches0
    # the median of three regions: a stall of the host (it launches ~100 kernels per step) would otherwise own the figure
    ms = statistics.median([ms, time_loop(step, steps), time_loop(step, steps)])
    K.check_status(dev)
    flops = 2 * blocks * 6.0 * pairs * C * C
    return {"ms": ms, "tflops": flops / (ms * 1e-3) / 1e12, "flops_per_step": flops, "n_voxels": int(coords.shape[0]), "pairs": pairs,
            "launches": launches}


def sharded_batch_steps(dev, world: int, rank: int, steps: int, warmup: int = 3):
    """The high-resolution batch (8 shells at RES=1024, radius scale 0.8 + 0.2 u,
    C=64 fp16): whole samples are dealt to the ranks (LPT by expected voxel
    count), every rank builds its own cache and runs fwd + bwd on its samples,
    the fp32 weight/bias gradient is all-reduced once per step.  Strong scaling:
    the batch is fixed.  Returns this rank's figures (ms of ``steps`` steps, build ms, voxels, pairs, launches)."""
    import torch.distributed as dist

    from flexgemm_b200 import sharding, workloads
    from flexgemm_b200.kernels import cuda as K
    from flexgemm_b200.ops.spconv import SubMConv3dFunction as F
    B, res, C = 8, 1024, 64
    g = torch.Generator().manual_seed(4)
    scales = [0.8 + 0.2 * float(u) for u in torch.rand(B, generator=g)]
    expected = [int(1e6 * s * s) for s in scales]          # shell area ~ radius^2: enough to balance the deal
    mine = sharding.assign_samples(expected, world)[rank]
    coords = workloads.shell_coords_torch(res, len(mine), [scales[i] for i in mine], device=dev)
    n = coords.shape[0]
    shape = torch.Size((max(len(mine), 1), C, res, res, res))
    gg = torch.Generator(device=dev).manual_seed(100 + rank)
    feats = torch.randn(n, C, generator=gg, device=dev, dtype=torch.float32).half()
    gw_ = torch.Generator().manual_seed(4)
    weight = (torch.randn(C, 3, 3, 3, C, generator=gw_) / (27 * C) ** 0.5).half().to(dev)   # identical on every rank
    bias = torch.randn(C, generator=gw_).half().to(dev)
    gout = torch.ones(n, C, dtype=torch.float16, device=dev)
    map_ms, cache = time_map_build(coords, shape, 3, warmup=2)
    pairs = int(cache["valid_signal_i"].shape[0])
    cache.block_order(K.conv_tile_rows())

    def step():
        out = F._sparse_submanifold_conv_forward(feats, cache, weight, bias)
        return out, sharding.sharded_backward(gout, feats, cache, weight, bias)

    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    K.check_status(dev)
    launches0 = K.launch_count
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        step()
    b.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    K.check_status(dev)
    return {"ms_total": a.elapsed_time(b), "map_ms": map_ms, "n": n, "pairs": pairs, "launches": K.launch_count - launches0,
            "scales": scales, "C": C}


def sharded_batch_report(dev, world: int, rank: int, steps: int):
    import torch.distributed as dist
    r = sharded_batch_steps(dev, world, rank, steps)
    stats = torch.tensor([r["ms_total"], r["map_ms"], float(r["n"]), float(r["pairs"])], dtype=torch.float64, device=dev)
    mx, sm = stats.clone(), stats.clone()
    if world > 1:
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        per_rank = [torch.zeros_like(stats) for _ in range(world)]
        dist.all_gather(per_rank, stats)
        voxels = [int(t[2].item()) for t in per_rank]
    else:
        voxels = [r["n"]]
    ms_step = mx[0].item() / steps
    total_pairs, total_n = sm[3].item(), sm[2].item()
    C = r["C"]
    return {"metric": "submconv fwd+bwd useful TFLOP/s (C=64 fp16, batch of 8 shells at RES=1024, sample-sharded)",
            "value": 6.0 * total_pairs * C * C / (ms_step * 1e-3) / 1e12, "unit": "TFLOP/s", "scaling": "strong", "ms_per_step": ms_step,
            "steps": steps, "n_voxels": int(total_n), "pairs": int(total_pairs), "per_rank_voxels": voxels,
            "load_balance_bound": total_n / max(mx[2].item(), 1.0), "map_build_ms": mx[1].item(),
            "scales": [round(s, 3) for s in r["scales"]], "launches": r["launches"]}


# --------------------------------------------------------------------------- the headline arm
def run_gpu_arm(args):
    import torch.distributed as dist

    from flexgemm_b200 import sharding, workloads
    from flexgemm_b200.kernels import cuda as K
    from flexgemm_b200.ops import spconv
    from flexgemm_b200.ops.spconv import SubMConv3dFunction as F

    world, rank, local_rank = dist_env()
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} does not match WORLD_SIZE {world}")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    peaks = load_peaks()
    spconv.set_algorithm(spconv.Algorithm.MASKED_IMPLICIT_GEMM_SPLITK)
    warmup = max(args.warmup, 3)
    reps = max(args.repeats, 1)

    # one sample per rank; every rank draws the same shell, its own features
    def rank_inputs(r):
        c, f, _, _, shp = workloads.make_problem(RES, CI, CO, torch.float16, seed=2 + r)
        return c, f, shp

    coords_h, feats_h, shape = rank_inputs(rank)
    g = torch.Generator().manual_seed(2)
    weight_h = (torch.randn(CO, 3, 3, 3, CI, generator=g) / (27 * CI) ** 0.5).half()   # identical on every rank
    bias_h = torch.randn(CO, generator=g).half()
    coords_h, feats_h = coords_h.pin_memory(), feats_h.pin_memory()
    coords, feats = coords_h.to(dev), feats_h.to(dev)
    weight, bias = weight_h.to(dev), bias_h.to(dev)
    n = coords.shape[0]
    gout = torch.ones(n, CO, dtype=torch.float16, device=dev)   # d(out.sum())/d(out)

    # ---- neighbour-map build ------------------------------------------------
    map_ms, cache = time_map_build(coords, shape, max(args.steps, 5), warmup)
    pairs = int(cache["valid_signal_i"].shape[0])
    flops_step = 6.0 * pairs * CI * CO
    tile = K.conv_tile_rows()
    cache.block_order(tile)
    f_req = feats.detach().requires_grad_(True)
    w_req = weight.detach().requires_grad_(True)
    b_req = bias.detach().requires_grad_(True)

    def step():
        out = F._sparse_submanifold_conv_forward(feats, cache, weight, bias)
        if world > 1:
            return out, sharding.sharded_backward(gout, feats, cache, weight, bias)
        return out, F._sparse_submanifold_conv_backward(gout, f_req, cache, w_req, b_req)

    def timed_region(steps):
        """K steps between a barrier + synchronize on both sides; device time, max over ranks."""
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            step()
        b.record()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        t = torch.tensor([a.elapsed_time(b)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    K.check_status(dev)
    sampler = ClockSampler(local_rank).start() if rank == 0 else None
    launches0 = K.launch_count
    # the part draws more than its power limit at full clocks, which holds for some tens of milliseconds only: an idle
    # pause before every repeat keeps each one in the short-burst regime the measured peak was taken in (the loop of a
    # second or more under the power cap is reported separately, see `sustained`)
    region_ms = []
    for _ in range(reps):
        time.sleep(args.pause)
        region_ms.append(timed_region(args.steps))
    launches = (K.launch_count - launches0) // reps          # of one timed region of K steps
    clocks = sampler.stop() if rank == 0 else None
    K.check_status(dev)
    per_step = sorted(t / args.steps for t in region_ms)
    ms_step = statistics.median(per_step)
    value = flops_step * world / (ms_step * 1e-3) / 1e12
    repeats = {"n": len(per_step), "steps_each": args.steps, "ms_per_step_median": ms_step, "ms_per_step_min": per_step[0],
               "ms_per_step_max": per_step[-1], "idle_pause_s_before_each": args.pause}

    roofline = None
    if rank == 0:
        # ---- per-kernel times for the roofline (rank 0), taken straight after the headline region: the same short-burst
        # regime as that region and as the measured peak (a loop of seconds runs under the power cap, see `sustained`)
        w_cvc = weight.reshape(CO, 27, CI)
        masks, order = cache.tile_masks(tile), cache.block_order(tile)
        it = max(args.steps, 10)

        def burst(fn):
            """median of `reps` short loops, each after an idle pause (same regime as the headline region)"""
            vals = []
            for _ in range(reps):
                time.sleep(args.pause)
                fn()
                vals.append(time_loop(fn, it))
            return statistics.median(vals)

        t_fprop = burst(lambda: K.conv_fprop(feats, w_cvc, bias, cache["neighbor_map"], cache["sorted_idx"], masks, order))
        t_dgrad = burst(lambda: K.conv_dgrad(gout, w_cvc, cache["neighbor_map"], cache["sorted_idx"], masks, order))
        t_wgrad = burst(lambda: K.conv_wgrad(gout, feats, cache["valid_signal_i"], cache["valid_signal_o"], cache["valid_signal_seg"],
                                             block_offsets=cache["pair_block_offsets"]))
        kernels = {"fprop": t_fprop, "dgrad": t_dgrad, "wgrad": t_wgrad}
        dom = max(kernels, key=kernels.get)
        pass_flops = 2.0 * pairs * CI * CO
        achieved = pass_flops / (kernels[dom] * 1e-3) / 1e12
        peak_tf = float(peaks["bf16_tflops"])
        roofline = {"bound": "tensor", "kernel": dom, "achieved": achieved, "peak": peak_tf, "unit": "TFLOP/s",
                    "frac": achieved / peak_tf, "traffic": NCU_DRAM_TRAFFIC["bytes"].get(dom),
                    "traffic_unit": "bytes per launch (ncu dram__bytes_read.sum + dram__bytes_write.sum)",
                    "traffic_from_capture_of_commit": NCU_DRAM_TRAFFIC["commit"],
                    "algorithmic_flops_per_launch": pass_flops, "peak_source": peaks["source"],
                    "ms": {k: round(v, 4) for k, v in kernels.items()},
                    "tflops": {k: round(pass_flops / (v * 1e-3) / 1e12, 1) for k, v in kernels.items()},
                    "frac_each": {k: round(pass_flops / (v * 1e-3) / 1e12 / peak_tf, 4) for k, v in kernels.items()},
                    "step_frac": round(value / world / peak_tf, 4)}

    # ---- end to end through the public API, host buffers ---------------------
    e2e_steps = max(3, min(args.steps, 10))
    loss_h = torch.empty(1, dtype=torch.float32).pin_memory()
    gw_h = torch.empty(weight.shape, dtype=torch.float16).pin_memory()
    copy_stream = torch.cuda.Stream(device=dev)

    def start_copies():
        """Queues one step's host-to-device copies on the copy stream: coordinates first (the
        neighbour cache needs only them), then the 32x larger features."""
        main = torch.cuda.current_stream(dev)
        with torch.cuda.stream(copy_stream):
            c = coords_h.to(dev, non_blocking=True)
            c_ready = torch.cuda.Event()
            c_ready.record(copy_stream)
            f = feats_h.to(dev, non_blocking=True)
            f_ready = torch.cuda.Event()
            f_ready.record(copy_stream)
        c.record_stream(main)
        f.record_stream(main)
        return c, c_ready, f, f_ready

    def e2e_run(iters: int):
        """``iters`` steps through the public API.  Every step's inputs come from pinned host memory
        and its loss and weight gradient go back to the host; as an input pipeline would, the copies of
        step k+1 are queued while step k computes."""
        main = torch.cuda.current_stream(dev)
        pending = start_copies()
        for k in range(iters):
            c, c_ready, f, f_ready = pending
            if k + 1 < iters:
                pending = start_copies()
            main.wait_event(c_ready)
            cache_e = F._compute_neighbor_cache(c, shape, (3, 3, 3), (1, 1, 1), True)
            main.wait_event(f_ready)
            f.requires_grad_(True)
            w = weight.detach().requires_grad_(True)
            bb = bias.detach().requires_grad_(True)
            out, _ = spconv.sparse_submanifold_conv3d(f, c, shape, w, bb, neighbor_cache=cache_e)
            loss = out.float().sum()
            loss.backward()
            gw = w.grad
            if world > 1:
                dist.all_reduce(gw)
            loss_h.copy_(loss.detach().reshape(1), non_blocking=True)
            gw_h.copy_(gw, non_blocking=True)

    e2e_run(2)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    # the host is in this loop (one round trip per cache build), so a timed region of a few steps is exposed to host
    # jitter: the region is repeated like the headline's and the median reported
    e2e_samples = []
    for _ in range(max(1, args.repeats)):
        ea, eb = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ea.record()
        e2e_run(e2e_steps)
        eb.record()
        torch.cuda.synchronize()
        t = torch.tensor([ea.elapsed_time(eb) / e2e_steps], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_samples.append(t.item())
    e2e_ms = statistics.median(e2e_samples)
    e2e_value = flops_step * world / (e2e_ms * 1e-3) / 1e12
    h2d = coords_h.numel() * 4 + feats_h.numel() * 2
    d2h = 4 + gw_h.numel() * 2

    def copies_only():
        """One step's host-to-device copies and nothing else: what the host side can feed."""
        _, _, _, f_ready = start_copies()
        torch.cuda.current_stream(dev).wait_event(f_ready)

    copies_only()
    if world > 1:
        dist.barrier()
    h2d_ms = torch.tensor([time_loop(copies_only, 5)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(h2d_ms, op=dist.ReduceOp.MAX)
    h2d_gbs = h2d / (h2d_ms.item() * 1e-3) / 1e9

    # ---- a loop of at least a second, against the sustained peak --------------
    sustained = None
    if not args.quick:
        n_sus = max(int(1100.0 / ms_step), args.steps)
        s2 = ClockSampler(local_rank).start() if rank == 0 else None
        sus_ms = timed_region(n_sus) / n_sus
        sus_clocks = s2.stop() if rank == 0 else None
        sus_tf = flops_step * world / (sus_ms * 1e-3) / 1e12
        peak_sus = float(peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"]))
        sustained = {"steps": n_sus, "ms_per_step": sus_ms, "value": sus_tf, "unit": "TFLOP/s", "peak_sustained": peak_sus,
                     "frac_per_gpu": sus_tf / world / peak_sus, "clocks": sus_clocks, "peak_source": peaks["source"]}

    # ---- N > 1: every phase alone, and the reduced gradient against the sum of the local ones ----
    phases = allreduce_check = None
    if world > 1:
        w_cvc = weight.reshape(CO, 27, CI)
        masks, order = cache.tile_masks(tile), cache.block_order(tile)
        nw = CO * 27 * CI
        flat = torch.empty(nw + CO, dtype=torch.float32, device=dev)

        def ph_fprop():
            K.conv_fprop(feats, w_cvc, bias, cache["neighbor_map"], cache["sorted_idx"], masks, order)

        def ph_wgrad():
            K.conv_wgrad(gout, feats, cache["valid_signal_i"], cache["valid_signal_o"], cache["valid_signal_seg"], want_f32=True,
                         want_dtype=False, block_offsets=cache["pair_block_offsets"], out_f32=flat[:nw])
            K.bias_grad(gout, want_f32=True, want_dtype=False, out_f32=flat[nw:])

        def ph_allreduce():
            dist.all_reduce(flat)

        def ph_dgrad():
            K.conv_dgrad(gout, w_cvc, cache["neighbor_map"], cache["sorted_idx"], masks, order)

        def ph_cast():
            K.cast_from_f32(flat, torch.float16)

        names = (("fprop_ms", ph_fprop), ("wgrad_bias_ms", ph_wgrad), ("allreduce_ms", ph_allreduce), ("dgrad_ms", ph_dgrad),
                 ("cast_ms", ph_cast))
        vals = []
        for _, fn in names:
            fn()
            dist.barrier()
            vals.append(time_loop(fn, max(args.steps, 10)))
        tv = torch.tensor(vals, dtype=torch.float64, device=dev)
        dist.all_reduce(tv, op=dist.ReduceOp.MAX)
        phases = {k: round(v, 4) for (k, _), v in zip(names, tv.tolist())}
        phases["sum_ms"] = round(sum(tv.tolist()), 4)
        phases["step_ms"] = round(ms_step, 4)
        phases["note"] = ("each phase timed alone on every rank (max over ranks); in a step the all-reduce overlaps dgrad and the "
                          "bias gradient overlaps wgrad")

        # what NCCL returns vs the sum of every rank's local gradient, recomputed on rank 0.  Compared in fp32, before the
        # cast: with grad_out = 1 the bias gradient is the voxel count, which fp16 cannot hold once several ranks are added.
        ph_wgrad()
        dist.all_reduce(flat)
        _, (_, gw_step, _) = step()                      # and the fp16 weight gradient a real step hands back
        torch.cuda.synchronize()
        if rank == 0:
            tot = torch.zeros(nw + CO, dtype=torch.float64, device=dev)
            for r in range(world):
                _, f_r, _ = rank_inputs(r)
                f_r = f_r.to(dev)
                _, gw32 = K.conv_wgrad(gout, f_r, cache["valid_signal_i"], cache["valid_signal_o"], cache["valid_signal_seg"],
                                       want_f32=True, want_dtype=False, block_offsets=cache["pair_block_offsets"])
                _, gb32 = K.bias_grad(gout, want_f32=True, want_dtype=False)
                tot[:nw] += gw32.reshape(-1).double()
                tot[nw:] += gb32.double()

            def rel(a, b):
                return (a.double() - b).abs().max().item() / max(b.abs().max().item(), 1e-30)

            err_w, err_b = rel(flat[:nw], tot[:nw]), rel(flat[nw:], tot[nw:])
            err_step = rel(gw_step.reshape(-1), tot[:nw])
            allreduce_check = {"max_rel_err": max(err_w, err_b), "grad_weight_f32": err_w, "grad_bias_f32": err_b,
                               "grad_weight_f16_of_a_step": err_step, "ranks": world,
                               "bound": "fp32 sums in a different order: <= 1e-5; after the cast to fp16: <= 1e-3",
                               "how": "rank 0 regenerates every rank's seeded features, computes each local fp32 gradient with "
                                      "the same kernels and adds them in fp64; compared with the all-reduced fp32 buffer"}
        dist.barrier()

    # ---- the sharded high-resolution batch (all ranks) ------------------------
    sharded = None
    if not args.quick:
        del f_req, w_req, b_req
        K.release_workspaces()
        torch.cuda.empty_cache()
        sharded = sharded_batch_report(dev, world, rank, steps=3 if world == 1 else 5)
        K.release_workspaces()
        torch.cuda.empty_cache()

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    both = map_build_report(coords, shape, peaks, max(args.steps, 5))
    map_bytes = both["sorted"]["algorithmic_bytes"]
    map_gbs = map_bytes / (map_ms * 1e-3) / 1e9
    roofline_map = {"bound": "hbm", "achieved": map_gbs, "peak": float(peaks["hbm_gbs"]), "unit": "GB/s",
                    "frac": map_gbs / float(peaks["hbm_gbs"]), "traffic": None, "algorithmic_bytes": map_bytes,
                    "peak_source": peaks["source"], "hash_path": both["hash"]}

    extra = {}
    if world == 1 and not args.quick:
        del cache
        K.release_workspaces()
        torch.cuda.empty_cache()
        big = workloads.shell_coords_torch(1024, 2, [1.0, 1.0], device=dev)
        extra["map_build_res1024"] = map_build_report(big, torch.Size((2, 64, 1024, 1024, 1024)), peaks, 5)
        del big
        K.release_workspaces()
        torch.cuda.empty_cache()
        extra["sweep"] = sweep_report(dev, peaks)
        K.release_workspaces()
        torch.cuda.empty_cache()
        unf = residual_stack_steps(dev, False, 5)
        fus = residual_stack_steps(dev, True, 5)
        extra["residual_stack"] = {
            "workload": f"8 x ([conv, SiLU, conv] + skip), C=512 bf16, 4 x RES=64, N={unf['n_voxels']} voxels, L={unf['pairs']} pairs "
                        "per conv, fwd+bwd of the mean, shared cache",
            "unfused": {"ms": round(unf["ms"], 3), "tflops": round(unf["tflops"], 1), "frac": round(unf["tflops"] / peak_tf, 4)},
            "fused": {"ms": round(fus["ms"], 3), "tflops": round(fus["tflops"], 1), "frac": round(fus["tflops"] / peak_tf, 4)}}

    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        tf, ms, sample = cpu_explicit_steps(3, 1, threads)
        cpu = {"value": tf, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample, "ms_per_step": ms}

    line = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16",
        "data": "synthetic",
        "config": {"workload": f"submconv3d k3 fwd+bwd (dgrad+wgrad+bias grad), spherical shell RES={RES}, Ci=Co={CI}, fp16, "
                               f"one sample per GPU, N={n} voxels, L={pairs} pairs, neighbour cache reused",
                   "l2": "inputs (feats, grad_out, neighbour map, pair lists: ~200 MB) exceed the 126 MB L2; no flush",
                   "parallelism": f"sample-sharded dp{world}, one fp32 all-reduce of wgrad+bias grad per step" if world > 1 else "single GPU"},
        "repeats": repeats, "sustained": sustained,
        "map_build_ms": map_ms, "map_build_ms_hash": both["hash"]["ms"],
        "roofline": roofline, "roofline_map_build": roofline_map, "cpu_baseline": cpu,
        "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_ms, "ms_per_step_min": min(e2e_samples), "ms_per_step_max": max(e2e_samples),
                "repeats": len(e2e_samples), "steps_each": e2e_steps, "h2d_gbs_per_gpu": h2d_gbs, "h2d_gbs_aggregate": h2d_gbs * world,
                "h2d_note": "the copies alone, all ranks pulling from pinned host memory at once (slowest rank): a step through "
                            "host buffers cannot be faster than h2d_bytes_per_step / h2d_gbs_per_gpu",
                "includes": "per step: H2D of coords+feats from pinned memory on a copy stream (the next step's copies are queued "
                            "while the current step computes), neighbour-map build, fwd, bwd, D2H of loss and grad_weight"},
        "gpu_launches": launches, "clocks": clocks,
        "phases": phases, "allreduce_check": allreduce_check, "sharded_batch": sharded,
    }
    line.update(extra)
    emit(line)
    if world > 1:
        dist.destroy_process_group()


# --------------------------------------------------------------------------- side workloads run alone
def run_sharded_batch(args):
    import torch.distributed as dist

    from flexgemm_b200.ops import spconv
    world, rank, local_rank = dist_env()
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} does not match WORLD_SIZE {world}")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    spconv.set_algorithm(spconv.Algorithm.MASKED_IMPLICIT_GEMM_SPLITK)
    sampler = ClockSampler(local_rank).start() if rank == 0 else None
    rep = sharded_batch_report(dev, world, rank, args.steps)
    clocks = sampler.stop() if rank == 0 else None
    if rank == 0:
        emit({"metric": rep["metric"], "value": rep["value"], "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": 3,
              "ms_per_step": rep["ms_per_step"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16",
              "data": "synthetic",
              "config": {"workload": f"submconv3d k3 fwd+bwd, 8 spherical shells RES=1024 (scales {rep['scales']}), Ci=Co=64, fp16, "
                                     f"N={rep['n_voxels']} voxels, L={rep['pairs']} pairs, cache reused",
                         "l2": "per-rank inputs far exceed the 126 MB L2; no flush",
                         "parallelism": f"whole samples dealt to {world} rank(s), one fp32 all-reduce of wgrad+bias grad per step",
                         "per_rank_voxels": rep["per_rank_voxels"], "load_balance_bound": rep["load_balance_bound"]},
              "map_build_ms": rep["map_build_ms"], "gpu_launches": rep["launches"], "clocks": clocks})
    if world > 1:
        dist.destroy_process_group()


def run_map_build(args):
    """Neighbour-cache build alone at a size where HBM matters: two shells at
    RES=1024 (5.3 M voxels, 56 M pairs, 32-bit keys), rows in key order (the
    table-free path) or shuffled (``--unsorted``: the hash-table path)."""
    from flexgemm_b200 import workloads
    from flexgemm_b200.kernels import cuda as K
    from flexgemm_b200.ops import spconv
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    peaks = load_peaks()
    spconv.set_algorithm(spconv.Algorithm.MASKED_IMPLICIT_GEMM_SPLITK)
    B, res = 2, 1024
    coords = workloads.shell_coords_torch(res, B, [1.0] * B, device=dev)
    if args.unsorted:
        coords = coords[torch.randperm(coords.shape[0], generator=torch.Generator().manual_seed(1)).to(dev)].contiguous()
    n = coords.shape[0]
    shape = torch.Size((B, 64, res, res, res))
    launches0 = K.launch_count
    sampler = ClockSampler(dev.index).start()
    ms, cache = time_map_build(coords, shape, args.steps, max(args.warmup, 3))
    launches = (K.launch_count - launches0) // (args.steps + max(args.warmup, 3))
    clocks = sampler.stop()
    K.check_status(dev)
    pairs = int(cache["valid_signal_i"].shape[0])
    nbytes = map_build_bytes(n, pairs, spconv.HASHMAP_RATIO)
    gbs = nbytes / (ms * 1e-3) / 1e9
    peak = float(peaks["hbm_gbs"])
    emit({
        "metric": "neighbor-cache build, algorithmic GB/s (2 shells at RES=1024)", "value": gbs, "unit": "GB/s", "n_gpus": 1,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "u32", "data": "synthetic",
        "config": {"workload": f"hash/neighbour map + sort + pair lists, N={n} voxels, L={pairs} pairs, 32-bit keys, "
                               f"rows {'shuffled (hash-table path)' if args.unsorted else 'in key order (table-free path)'}",
                   "l2": "working set (coords, table, map, lists: ~1.5 GB) far exceeds the 126 MB L2; no flush"},
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak, "traffic": None,
                     "algorithmic_bytes": nbytes, "peak_source": peaks["source"]},
        "gpu_launches": launches, "clocks": clocks})


def run_residual_stack(args):
    from flexgemm_b200.ops import spconv
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    peaks = load_peaks()
    spconv.set_algorithm(spconv.Algorithm.MASKED_IMPLICIT_GEMM_SPLITK)
    sampler = ClockSampler(dev.index).start()
    r = residual_stack_steps(dev, args.fused, args.steps, max(args.warmup, 3))
    clocks = sampler.stop()
    peak = float(peaks["bf16_tflops"])
    emit({
        "metric": "residual stack fwd+bwd useful TFLOP/s (16 submconvs, C=512 bf16, 4 x RES=64)", "value": r["tflops"], "unit": "TFLOP/s",
        "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": r["ms"], "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"8 x ([conv, SiLU, conv] + skip), N={r['n_voxels']} voxels, L={r['pairs']} pairs per conv, shared cache; "
                               f"elementwise work {'in the conv epilogues' if args.fused else 'as torch kernels'}",
                   "l2": "activations of one layer (41 MB) fit the 126 MB L2; no flush: the stack streams 16 layers of them"},
        "roofline": {"bound": "tensor", "achieved": r["tflops"], "peak": peak, "unit": "TFLOP/s", "frac": r["tflops"] / peak, "traffic": None,
                     "algorithmic_flops_per_step": r["flops_per_step"], "peak_source": peaks["source"]},
        "gpu_launches": r["launches"], "clocks": clocks})


def run_pipeline_microbench(args):
    """What one SM sustains of an fprop stage's operand streams and MMAs (kernels.cuda.microbench_pipeline): the
    numbers behind the tensor-pipe ceiling of fprop / dgrad."""
    import torch
    from flexgemm_b200.kernels import cuda as K
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    n_rows, c = 163736, 256                       # the headline workload's feature matrix (84 MB) and weights (3.5 MB)
    rows = torch.zeros(n_rows, c, dtype=torch.float16, device=dev)
    dense = torch.zeros(27 * c * c, dtype=torch.float16, device=dev)
    iters = 2000
    T, G, M, C, G4, P, L = K.MB_TMA, K.MB_GATHER, K.MB_MMA, K.MB_COUPLED, K.MB_GATHER4, K.MB_PAIR, K.MB_LEAN
    M64, ST, SB128, SB512 = K.MB_M64, K.MB_STORE, K.MB_STORE_BULK128, K.MB_STORE_BULK512
    cases = [("mma alone", M, 3, 3, 0), ("mma alone, 64 x 256 x 16 instead of 128 x 256 x 16", M | M64, 3, 3, 0),
             ("mma alone, 128 idle cycles before each stage", M, 3, 3, 128),
             ("mma alone, 256 idle cycles before each stage", M, 3, 3, 256),
             ("tma alone", T, 3, 3, 0), ("gather alone (cp.async)", G, 3, 3, 0), ("gather alone (TMA gather4)", G | G4, 3, 3, 0),
             ("tma + gather, independent", T | G, 3, 3, 0), ("mma + tma + gather, independent", M | T | G, 3, 3, 0),
             ("coupled: mma + tma + gather, 2 stages", C | M | T | G, 2, 2, 0), ("coupled: mma + tma + gather, 3 stages", C | M | T | G, 3, 3, 0),
             ("coupled: mma + tma + gather, 5 + 2 stages", C | M | T | G, 5, 2, 0),
             ("coupled, lean MMA lane: mma + tma", L | C | M | T, 3, 3, 0), ("coupled, lean MMA lane: mma + gather", L | C | M | G, 3, 3, 0),
             ("coupled, lean MMA lane: mma + tma + gather, 2 stages", L | C | M | T | G, 2, 2, 0),
             ("coupled, lean MMA lane: mma + tma + gather, 3 stages", L | C | M | T | G, 3, 3, 0),
             ("coupled, lean MMA lane: mma + tma + gather, 5 + 2 stages", L | C | M | T | G, 5, 2, 0),
             ("CTA pairs, 3 stages", P, 3, 3, 0), ("CTA pairs, 4 stages", P, 4, 4, 0),
             ("output stream alone: 16-byte stores, four 128-byte lines per warp instruction", ST, 3, 3, 0),
             ("output stream alone: bulk async copies of 128 bytes", SB128, 3, 3, 0),
             ("output stream alone: bulk async copies of 512-byte rows", SB512, 3, 3, 0),
             ("mma + output stream (16-byte stores)", M | ST, 3, 3, 0)]
    sampler = ClockSampler(dev.index).start()
    out, launches = [], 0
    for name, mode, sa, sb, delay in cases:
        best, ctr = None, None
        for _ in range(max(args.warmup, 1) + max(1, min(args.steps, 5))):
            time.sleep(0.05)                       # every launch in the short-burst clock regime
            ms, c8 = K.microbench_pipeline(mode, rows, dense, iters, sa, sb, delay)
            launches += 1
            if best is None or ms < best:
                best, ctr = ms, c8
        pair = bool(mode & P)
        b_chunk = 16384 if pair else 32768
        moved = ((32768 if mode & (G | ST | SB128 | SB512) or pair else 0) + (b_chunk if mode & T or pair else 0)) * iters
        rec = {"case": name, "us_per_stage": round(best * 1e3 / iters, 4), "moved_gbs_per_sm": round(moved / best * 1e-6, 1)}
        if mode & M or pair:
            rec["mma_frac_of_nominal"] = round(iters * 8 * 128 / 1.965e6 / best, 3)   # 8 MMAs x 128 cycles at 1965 MHz
            if mode & C or pair:
                rec["mma_lane"] = {"wait_dense_cycles": ctr[0], "waits_dense": ctr[1], "wait_gathered_cycles": ctr[2], "waits_gathered": ctr[3],
                                   "loop_cycles": ctr[4], "stages": iters}
        out.append(rec)
    clocks = sampler.stop()
    head = next(r for r in out if r["case"].startswith("coupled, lean MMA lane: mma + tma + gather, 3"))
    emit({"metric": "pipeline microbenchmark: time per fprop stage on one SM (64 KB of operands in, 8 MMAs 128x256x16)",
          "value": head["us_per_stage"], "unit": "us", "n_gpus": 1, "steps": iters, "warmup": max(args.warmup, 1), "ms_per_step": head["us_per_stage"] * 1e-3,
          "higher_is_better": False, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
          "config": {"workload": "per SM and stage: 256 random rows x 128 B gathered from an 84 MB matrix, 32 KB by TMA from a 3.5 MB buffer, "
                                 "8 MMAs 128x256x16; all 148 SMs at once; best of a few launches per case",
                     "l2": "the 84 MB matrix and the 3.5 MB buffer are L2-resident after the first launch (an upper bound for the conv kernel, whose "
                           "gathers hit L2 78 % of the time)"},
          "cases": out, "gpu_launches": launches, "clocks": clocks})


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--repeats", type=int, default=5, help="how many times the timed region of --steps steps is run (median reported)")
    ap.add_argument("--pause", type=float, default=0.5, help="idle seconds before each repeat (keeps every repeat in the short-burst regime)")
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--quick", action="store_true", help="headline workload only: no sustained loop, sweep, residual stack, RES=1024 runs")
    ap.add_argument("--workload", default="res256", choices=["res256", "res1024_batch8", "res1024_map", "residual_stack", "pipeline_microbench"],
                    help="res256: the headline single-sample workload (default); res1024_batch8: the sharded high-resolution "
                         "batch; res1024_map: the neighbour-cache build alone at a size where HBM matters; residual_stack: 16 convs "
                         "with SiLU and skip additions between them; pipeline_microbench: operand streams and MMAs of one fprop stage per SM")
    ap.add_argument("--unsorted", action="store_true", help="res1024_map: shuffle the rows (hash-table path)")
    ap.add_argument("--fused", action="store_true", help="residual_stack: SiLU and skip additions in the conv epilogues")
    args = ap.parse_args()
    claim_stdout()
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.workload == "res1024_batch8":
        run_sharded_batch(args)
    elif args.workload == "res1024_map":
        run_map_build(args)
    elif args.workload == "residual_stack":
        run_residual_stack(args)
    elif args.workload == "pipeline_microbench":
        run_pipeline_microbench(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
