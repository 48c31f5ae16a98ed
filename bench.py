"""Benchmark of the submanifold-conv3d hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One step = forward + backward (dgrad, wgrad, bias grad) of one 3x3x3
submanifold convolution on the headline workload: a spherical shell at
RES=256, C=256 -> 256, fp16, one sample per GPU (weak scaling: with N GPUs the
batch holds N samples, one per rank, and the weight/bias gradient is summed
with one NCCL all-reduce per step).  The reported value is useful TFLOP/s,
6 * L * Ci * Co per step with L = number of valid (voxel, offset) pairs.

Printed JSON (one line, rank 0): the metric and, beside it, the neighbour-map
build time, a roofline object for the dominant kernel and for the map build,
the CPU baseline (the explicit gather-GEMM-scatter algorithm of the reference,
restated in oracle/, timed on this host's cores on a bounded slab of the same
workload), an end-to-end figure through the public API with host buffers, the
number of kernels launched and the SM clocks sampled during the timed region.

--impl reference times that CPU algorithm alone, with all host threads.

--workload res1024_batch8 runs the high-resolution sharded batch instead (8
shells at RES=1024, C=64, fp16, whole samples dealt to the ranks, strong
scaling); its line carries the metric, the per-rank balance and the clocks only.
--workload res1024_map [--unsorted] times the neighbour-cache build alone on two
shells at RES=1024 and reports its algorithmic GB/s against the HBM peak.
--workload residual_stack [--fused] times a stack of 8 residual blocks (16 convs,
C=512, bf16) forward + backward, with the elementwise work between the convs as
torch kernels or in the conv kernels' epilogue.
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
# dram__bytes_read.sum + dram__bytes_write.sum per launch at this workload, from the ncu capture summarised in
# profiles/subm_igemm_and_wgrad_res256_c256_fp16.md
NCU_DRAM_TRAFFIC_BYTES = {"fprop": 291.9e6, "dgrad": 291.4e6, "wgrad": 522.4e6}


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
    line = {
        "impl": "reference", "metric": METRIC, "value": tflops, "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"submconv3d k3 fwd+bwd, spherical shell RES={RES}, Ci=Co={CI}, explicit gather-GEMM-scatter on host cores",
                   "sample": sample},
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


# --------------------------------------------------------------------------- GPU arm
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


def run_gpu_arm(args):
    import torch.distributed as dist

    from flexgemm_b200 import sharding, workloads
    from flexgemm_b200.kernels import cuda as K
    from flexgemm_b200.ops import spconv
    from flexgemm_b200.ops.spconv import SubMConv3dFunction as F

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} does not match WORLD_SIZE {world}")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    peaks = load_peaks()
    spconv.set_algorithm(spconv.Algorithm.MASKED_IMPLICIT_GEMM_SPLITK)

    # one sample per rank; every rank draws the same shell, its own features
    coords_h, feats_h, weight_h, bias_h, shape = workloads.make_problem(RES, CI, CO, torch.float16, seed=2 + rank)
    g = torch.Generator().manual_seed(2)
    weight_h = (torch.randn(CO, 3, 3, 3, CI, generator=g) / (27 * CI) ** 0.5).half()   # identical on every rank
    bias_h = torch.randn(CO, generator=g).half()
    coords_h, feats_h = coords_h.pin_memory(), feats_h.pin_memory()
    coords, feats = coords_h.to(dev), feats_h.to(dev)
    weight, bias = weight_h.to(dev), bias_h.to(dev)
    n = coords.shape[0]
    gout = torch.ones(n, CO, dtype=torch.float16, device=dev)   # d(out.sum())/d(out)

    # ---- neighbour-map build ------------------------------------------------
    def build():
        return F._compute_neighbor_cache(coords, shape, (3, 3, 3), (1, 1, 1), True)

    for _ in range(max(args.warmup, 3)):
        cache = build()
    map_ms = time_loop(build, max(args.steps, 5))
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

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    K.check_status(dev)
    launches0 = K.launch_count
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(args.steps):
        step()
    b.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ms_total = a.elapsed_time(b)
    launches = K.launch_count - launches0
    clocks = sampler.stop() if rank == 0 else None
    K.check_status(dev)
    t = torch.tensor([ms_total], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = t.item() / args.steps
    value = flops_step * world / (ms_step * 1e-3) / 1e12

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
    ea, eb = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ea.record()
    e2e_run(e2e_steps)
    eb.record()
    torch.cuda.synchronize()
    e2e_ms = ea.elapsed_time(eb) / e2e_steps
    t = torch.tensor([e2e_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_value = flops_step * world / (t.item() * 1e-3) / 1e12
    h2d = coords_h.numel() * 4 + feats_h.numel() * 2
    d2h = 4 + gw_h.numel() * 2

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- per-kernel times for the roofline (rank 0) --------------------------
    w_cvc = weight.reshape(CO, 27, CI)
    masks, order = cache.tile_masks(tile), cache.block_order(tile)
    it = max(args.steps, 10)
    t_fprop = time_loop(lambda: K.conv_fprop(feats, w_cvc, bias, cache["neighbor_map"], cache["sorted_idx"], masks, order), it)
    t_dgrad = time_loop(lambda: K.conv_dgrad(gout, w_cvc, cache["neighbor_map"], cache["sorted_idx"], masks, order), it)
    t_wgrad = time_loop(lambda: K.conv_wgrad(gout, feats, cache["valid_signal_i"], cache["valid_signal_o"], cache["valid_signal_seg"],
                                             block_offsets=cache["pair_block_offsets"]), it)
    kernels = {"fprop": t_fprop, "dgrad": t_dgrad, "wgrad": t_wgrad}
    dom = max(kernels, key=kernels.get)
    pass_flops = 2.0 * pairs * CI * CO
    achieved = pass_flops / (kernels[dom] * 1e-3) / 1e12
    peak_tf = float(peaks["bf16_tflops"])
    roofline = {"bound": "tensor", "kernel": dom, "achieved": achieved, "peak": peak_tf, "unit": "TFLOP/s",
                "frac": achieved / peak_tf, "traffic": NCU_DRAM_TRAFFIC_BYTES.get(dom), "traffic_unit": "bytes per launch (ncu)",
                "algorithmic_flops_per_launch": pass_flops, "peak_source": peaks["source"],
                "ms": {k: round(v, 4) for k, v in kernels.items()},
                "tflops": {k: round(pass_flops / (v * 1e-3) / 1e12, 1) for k, v in kernels.items()}}
    V, k = 27, 4
    slots = int(spconv.HASHMAP_RATIO * n)
    map_bytes = (16 * n + k * slots + (k + 4) * n) + (16 * n + 13 * n * k + 4 * (pairs - n) // 2 + 4 * V * n) + \
                (4 * V * n + 4 * n + 8 * n + 8 * pairs)
    map_gbs = map_bytes / (map_ms * 1e-3) / 1e9
    roofline_map = {"bound": "hbm", "achieved": map_gbs, "peak": float(peaks["hbm_gbs"]), "unit": "GB/s",
                    "frac": map_gbs / float(peaks["hbm_gbs"]), "traffic": None, "algorithmic_bytes": map_bytes,
                    "peak_source": peaks["source"]}

    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        tf, ms, sample = cpu_explicit_steps(3, 1, threads)
        cpu = {"value": tf, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample, "ms_per_step": ms}

    line = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16",
        "data": "synthetic",
        "config": {"workload": f"submconv3d k3 fwd+bwd (dgrad+wgrad+bias grad), spherical shell RES={RES}, Ci=Co={CI}, fp16, "
                               f"one sample per GPU, N={n} voxels, L={pairs} pairs, neighbour cache reused",
                   "l2": "inputs (feats, grad_out, neighbour map, pair lists: ~200 MB) exceed the 126 MB L2; no flush",
                   "parallelism": f"sample-sharded dp{world}, one fp32 all-reduce of wgrad+bias grad per step" if world > 1 else "single GPU"},
        "map_build_ms": map_ms,
        "roofline": roofline, "roofline_map_build": roofline_map, "cpu_baseline": cpu,
        "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": t.item(), "includes": "per step: H2D of coords+feats from pinned memory on a copy stream (the next step's copies are queued while the current step computes), neighbour-map build, fwd, bwd, D2H of loss and grad_weight"},
        "gpu_launches": launches, "clocks": clocks,
    }
    emit(line)
    if world > 1:
        dist.destroy_process_group()


def run_sharded_batch(args):
    """The high-resolution sharded batch (8 shells at RES=1024, radius scale
    0.8 + 0.2 u, C=64 fp16): whole samples are dealt to the ranks (LPT by
    expected voxel count), every rank builds its own cache and runs fwd + bwd on
    its samples, the fp32 weight/bias gradient is all-reduced once per step.
    Strong scaling: the batch is fixed, ``value`` = useful FLOP of the whole batch
    / slowest rank's time."""
    import torch.distributed as dist

    from flexgemm_b200 import sharding, workloads
    from flexgemm_b200.kernels import cuda as K
    from flexgemm_b200.ops import spconv
    from flexgemm_b200.ops.spconv import SubMConv3dFunction as F

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} does not match WORLD_SIZE {world}")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    spconv.set_algorithm(spconv.Algorithm.MASKED_IMPLICIT_GEMM_SPLITK)
    B, res, C = 8, 1024, 64
    g = torch.Generator().manual_seed(4)
    scales = [0.8 + 0.2 * float(u) for u in torch.rand(B, generator=g)]
    expected = [int(1e6 * s * s) for s in scales]          # shell area ~ radius^2: enough to balance the deal
    mine = sharding.assign_samples(expected, world)[rank]
    coords_h = torch.from_numpy(workloads.shell_coords(res, len(mine), [scales[i] for i in mine]))
    coords = coords_h.to(dev)
    n = coords.shape[0]
    shape = torch.Size((max(len(mine), 1), C, res, res, res))
    gg = torch.Generator(device=dev).manual_seed(100 + rank)
    feats = torch.randn(n, C, generator=gg, device=dev, dtype=torch.float32).half()
    gw_ = torch.Generator().manual_seed(4)
    weight = (torch.randn(C, 3, 3, 3, C, generator=gw_) / (27 * C) ** 0.5).half().to(dev)   # identical on every rank
    bias = torch.randn(C, generator=gw_).half().to(dev)
    gout = torch.ones(n, C, dtype=torch.float16, device=dev)

    def build():
        return F._compute_neighbor_cache(coords, shape, (3, 3, 3), (1, 1, 1), True)

    for _ in range(2):
        cache = build()
    map_ms = time_loop(build, 3)
    pairs = int(cache["valid_signal_i"].shape[0])
    cache.block_order(K.conv_tile_rows())

    def step():
        out = F._sparse_submanifold_conv_forward(feats, cache, weight, bias)
        return out, sharding.sharded_backward(gout, feats, cache, weight, bias)

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    K.check_status(dev)
    launches0 = K.launch_count
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(args.steps):
        step()
    b.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    launches = K.launch_count - launches0
    clocks = sampler.stop() if rank == 0 else None
    K.check_status(dev)
    stats = torch.tensor([a.elapsed_time(b), map_ms, float(n), float(pairs)], dtype=torch.float64, device=dev)
    mx, sm = stats.clone(), stats.clone()
    if world > 1:
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
    if rank == 0:
        ms_step = mx[0].item() / args.steps
        total_pairs, total_n = sm[3].item(), sm[2].item()
        value = 6.0 * total_pairs * C * C / (ms_step * 1e-3) / 1e12
        line = {
            "metric": "submconv fwd+bwd useful TFLOP/s (C=64 fp16, batch of 8 shells at RES=1024, sample-sharded)",
            "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16",
            "data": "synthetic",
            "config": {"workload": f"submconv3d k3 fwd+bwd, 8 spherical shells RES=1024 (scales {[round(s, 3) for s in scales]}), "
                                   f"Ci=Co=64, fp16, N={int(total_n)} voxels, L={int(total_pairs)} pairs, cache reused",
                       "l2": "per-rank inputs far exceed the 126 MB L2; no flush",
                       "parallelism": f"whole samples dealt to {world} rank(s), one fp32 all-reduce of wgrad+bias grad per step",
                       "max_rank_voxels": int(mx[2].item()), "load_balance_bound": total_n / max(mx[2].item(), 1.0)},
            "map_build_ms": mx[1].item(), "gpu_launches": launches, "clocks": clocks,
        }
        emit(line)
    if world > 1:
        dist.destroy_process_group()


def run_map_build(args):
    """Neighbour-cache build alone at a size where HBM matters: two shells at
    RES=1024 (5.3 M voxels, 56 M pairs, 32-bit keys), rows in key order (the
    table-free path) or shuffled (``--unsorted``: the hash-table path).  Reports
    the algorithmic bytes of the build per second against the measured HBM peak."""
    from flexgemm_b200 import workloads
    from flexgemm_b200.kernels import cuda as K
    from flexgemm_b200.ops import spconv
    from flexgemm_b200.ops.spconv import SubMConv3dFunction as F

    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    peaks = load_peaks()
    spconv.set_algorithm(spconv.Algorithm.MASKED_IMPLICIT_GEMM_SPLITK)
    B, res = 2, 1024
    coords_h = torch.from_numpy(workloads.shell_coords(res, B, [1.0] * B))
    if args.unsorted:
        coords_h = coords_h[torch.randperm(coords_h.shape[0], generator=torch.Generator().manual_seed(1))].contiguous()
    coords = coords_h.to(dev)
    n = coords.shape[0]
    shape = torch.Size((B, 64, res, res, res))

    def build():
        return F._compute_neighbor_cache(coords, shape, (3, 3, 3), (1, 1, 1), True)

    for _ in range(max(args.warmup, 3)):
        cache = build()
    K.check_status(dev)
    launches0 = K.launch_count
    sampler = ClockSampler(dev.index)
    sampler.start()
    ms = time_loop(build, args.steps)
    launches = K.launch_count - launches0
    clocks = sampler.stop()
    pairs = int(cache["valid_signal_i"].shape[0])
    V, k = 27, 4
    slots = int(spconv.HASHMAP_RATIO * n)
    nbytes = (16 * n + k * slots + (k + 4) * n) + (16 * n + 13 * n * k + 4 * (pairs - n) // 2 + 4 * V * n) + \
             (4 * V * n + 4 * n + 8 * n + 8 * pairs)
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
    """Residual stack: 8 blocks [conv, SiLU, conv] + skip on 4 shells at RES=64,
    C=512, bf16, one shared neighbour cache, forward + backward of the mean.
    ``--fused``: SiLU and the skip addition run in the conv kernels' epilogue
    (``sparse_submanifold_conv3d_fused``) instead of torch elementwise kernels."""
    from flexgemm_b200 import workloads
    from flexgemm_b200.kernels import cuda as K
    from flexgemm_b200.ops import spconv
    from flexgemm_b200.ops.spconv import SubMConv3dFunction as F

    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    peaks = load_peaks()
    spconv.set_algorithm(spconv.Algorithm.MASKED_IMPLICIT_GEMM_SPLITK)
    B, res, C, blocks = 4, 64, 512, 8
    dt = torch.bfloat16
    coords = torch.from_numpy(workloads.shell_coords(res, B, [1.0] * B)).to(dev)
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
            if args.fused:
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

    for _ in range(max(args.warmup, 3)):
        step()
    K.check_status(dev)
    launches0 = K.launch_count
    sampler = ClockSampler(dev.index)
    sampler.start()
    ms = time_loop(step, args.steps)
    launches = K.launch_count - launches0
    clocks = sampler.stop()
    K.check_status(dev)
    flops = 2 * blocks * 6.0 * pairs * C * C
    tf = flops / (ms * 1e-3) / 1e12
    peak = float(peaks["bf16_tflops"])
    emit({
        "metric": "residual stack fwd+bwd useful TFLOP/s (16 submconvs, C=512 bf16, 4 x RES=64)", "value": tf, "unit": "TFLOP/s",
        "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"8 x ([conv, SiLU, conv] + skip), N={coords.shape[0]} voxels, L={pairs} pairs per conv, shared cache; "
                               f"elementwise work {'in the conv epilogues' if args.fused else 'as torch kernels'}",
                   "l2": "activations of one layer (41 MB) fit the 126 MB L2; no flush: the stack streams 16 layers of them"},
        "roofline": {"bound": "tensor", "achieved": tf, "peak": peak, "unit": "TFLOP/s", "frac": tf / peak, "traffic": None,
                     "algorithmic_flops_per_step": flops, "peak_source": peaks["source"]},
        "gpu_launches": launches, "clocks": clocks})


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)  # 50 steps = 40 ms: long enough for a few dozen clock samples
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--workload", default="res256", choices=["res256", "res1024_batch8", "res1024_map", "residual_stack"],
                    help="res256: the headline single-sample workload (default); res1024_batch8: the sharded high-resolution "
                         "batch; res1024_map: the neighbour-cache build alone at a size where HBM matters; residual_stack: 16 convs "
                         "with SiLU and skip additions between them")
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
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
