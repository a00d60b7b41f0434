#!/usr/bin/env python3
"""Benchmark of the W4A4 hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--m M]

One step = one pass of the four Qwen3-8B linears (QKV 4096->6144, O 4096->4096, gate+up
4096->24576, down 12288->4096) over M tokens with per-group-128 scales: fused activation
quantise+pack followed by the W4A4 GEMM, i.e. what the linear method's ``apply`` does.  The
metric is GEMM throughput in TOPS (2*M*N*K per linear) over the whole step.  With N > 1 every
rank owns N/n output columns of each weight (no collective) and the value is the whole-job
aggregate.  Prints ONE JSON line on rank 0.

``--impl reference`` times the reference's own CPU formulation of the same path (fp32 quantise,
pack, int32 ``torch.matmul``, fp32 scales -> bf16) on the host cores, on a bounded row sample.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

SHAPES = [("qkv", 4096, 6144), ("o", 4096, 4096), ("gate_up", 4096, 24576), ("down", 12288, 4096)]
METRIC = "w4a4_gemm_tops_qwen3_8b_shapes_g128"
METRIC_CHANNEL = "w4a4_gemm_tops_qwen3_8b_shapes_per_channel"
UNIT = "TOPS"
GROUP = 128


_RESULT_FD = None


def claim_stdout() -> None:
    """Keep stdout to the one JSON line: libraries that write to file descriptor 1 themselves (NCCL prints its version
    there) are sent to stderr for the rest of the run, and the result goes to the descriptor saved here."""
    global _RESULT_FD
    sys.stdout.flush()
    _RESULT_FD = os.dup(1)
    os.dup2(2, 1)


def emit(line: dict) -> None:
    data = (json.dumps(line) + "\n").encode()
    if _RESULT_FD is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_RESULT_FD, data)


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            d = json.load(fh)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# --------------------------------------------------------------------------- #
# clocks
# --------------------------------------------------------------------------- #
class ClockSampler:
    FIELDS = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None

    def start(self):
        self.t_begin = None
        self.t_end = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.05)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        import datetime

        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                ts = datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                if self.t_begin is not None and not (self.t_begin - 0.05 <= ts <= self.t_end + 0.05):
                    continue  # keep only samples taken while the load was running
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        busy = sm
        return {"sm_mhz": statistics.median(busy), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


# --------------------------------------------------------------------------- #
# reference CPU formulation (bounded sample)
# --------------------------------------------------------------------------- #
def cpu_reference_step(rows: int, seed: int = 0):
    """The reference's torch CPU path on `rows` tokens of every linear: quantise as
    benchmark/benchmark_w4a8fp8.py:200-204, pack as int4_native_tc/profile_bottleneck.py:25-28,
    int32 torch.matmul + fp32 scales as benchmark/verify_int4_matmul_precision.py:23-29
    (per group, accumulated in fp32), bf16 result.  Returns (seconds, ops)."""
    from fp8_inference_toolkit_b200 import synthetic
    from oracle import w4a4_oracle as O  # CPU baseline leg: the one place the bench runs the oracle package

    total_t, total_ops = 0.0, 0
    for i, (_, K, N) in enumerate(SHAPES):
        x = synthetic.activations(rows, K, seed)
        w = synthetic.weights(N, K, seed + 1 + i)
        G = K // GROUP
        wq = w.float().reshape(N, G, GROUP)
        wa = wq.abs().amax(dim=2)
        ws = torch.where(wa == 0, torch.ones_like(wa), wa / 7.0)                     # int4_quant.cu:267 (zero group: scale 1)
        wc = torch.clamp(torch.round(wq / ws.unsqueeze(2)), -8, 7).to(torch.int32)  # weights: load time, untimed
        t0 = time.perf_counter()
        xq = x.float().reshape(rows, G, GROUP)
        xa = xq.abs().amax(dim=2)
        xd = torch.where(xa == 0, torch.ones_like(xa), xa / 7.0)                     # codes come from the un-floored absmax / 7
        xc = torch.clamp(torch.round(xq / xd.unsqueeze(2)), -8, 7).to(torch.int8)
        xs = (xa / 7.0).clamp(min=1.0 / (7.0 * 512.0))                               # returned scale: floor of int4_quant.cu:97,142
        packed = (xc[..., 0::2] & 0x0F) | ((xc[..., 1::2] & 0x0F) << 4)  # noqa: F841  (the pack step)
        acc = torch.zeros(rows, N, dtype=torch.float32)
        xi = xc.to(torch.int32)
        for g in range(G):
            part = O.int_gemm_int32_torch(xi[:, g], wc[:, g])
            acc += part.float() * xs[:, g].unsqueeze(1) * ws[:, g].unsqueeze(0)
        out = acc.to(torch.bfloat16)  # noqa: F841
        total_t += time.perf_counter() - t0
        total_ops += 2 * rows * N * K
    return total_t, total_ops


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # only this rank works: give it every host thread (a launcher may have pinned OMP_NUM_THREADS to 1)
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    cores = torch.get_num_threads()
    budget = 150.0  # seconds for the whole run
    t, ops = cpu_reference_step(2)
    per_row = max(t / 2, 1e-4)
    rows = int(max(1, min(args.m, budget / (args.steps + args.warmup) / per_row)))
    for _ in range(args.warmup):
        cpu_reference_step(rows)
    t_sum, ops_sum = 0.0, 0
    for _ in range(args.steps):
        t, ops = cpu_reference_step(rows)
        t_sum += t
        ops_sum += ops
    value = ops_sum / t_sum / 1e12
    sample = f"{rows} of {args.m} token rows of each of the 4 linears per step (activation quantise+pack, int32 torch.matmul per group, fp32 scales)"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": t_sum / args.steps * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "s4*s4->s32, f32 dequant",
        "data": "synthetic", "config": workload_config(args.m, args.gpus),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


def workload_config(M: int, n_gpus: int, per_channel: bool = False) -> dict:
    scales = "per-token / per-channel" if per_channel else "per-group-128"
    return {
        "workload": f"BASELINE configs[1]: dense W4A4 {scales} linears at Qwen3-8B shapes "
                    f"(K,N) in (4096,6144),(4096,4096),(4096,24576),(12288,4096), M={M} tokens; "
                    f"step = quantise+pack of the activations then the fused GEMM, for each shape"
                    + ("; the quantise of the next linear runs on a second stream under the GEMM" if n_gpus > 1 else ""),
        "M": M, "group_size": 0 if per_channel else GROUP, "n_split": n_gpus,
        "l2": "inputs larger than L2 (weights + activations + outputs of one step exceed 126 MB)",
    }


# --------------------------------------------------------------------------- #
# our arm
# --------------------------------------------------------------------------- #
def gemm_bytes(M, N, K):
    G = K // GROUP
    return M * K // 2 + N * K // 2 + 4 * G * (M + N) + 2 * M * N


def run_ours(args) -> None:
    import torch.distributed as dist

    import int4_native_tc as tc
    from fp8_inference_toolkit_b200 import ops, synthetic
    from fp8_inference_toolkit_b200.linear import W4A4Linear

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    M = args.m
    peaks = load_peaks()
    per_channel = args.scales == "channel"

    # ---- inputs resident in HBM: activations per shape, this rank's column slice of the weights
    layers, xs_dev = [], []
    for i, (name, K, N) in enumerate(SHAPES):
        assert N % world == 0
        n_loc = N // world
        w = synthetic.weights(N, K, seed=1 + i)[rank * n_loc:(rank + 1) * n_loc].to(dev)
        lin = W4A4Linear(K, n_loc, per_channel=per_channel, device=dev)
        lin.weight.data.copy_(w)
        lin.quantize_()
        layers.append(lin)
        xs_dev.append(synthetic.activations(M, K, seed=0, device=dev))
        del w
    outs = [torch.empty(M, l.out_features, dtype=torch.bfloat16, device=dev) for l in layers]
    ops_per_step = sum(2 * M * N * K for _, K, N in SHAPES)  # whole job, all ranks

    # With the output columns split over several GPUs every rank still quantises whole activations, so that part of
    # the step does not shrink with N.  It is HBM-bound while the GEMM is tensor/ALU-bound, and the four linears of a
    # step have independent inputs: from two GPUs on, the quantise of linear i + 1 runs on a second stream under the
    # GEMM of linear i (it fills the SMs that the GEMM's last wave leaves idle).
    overlap = world > 1
    quant_stream = torch.cuda.Stream(dev) if overlap else None

    def quantise(i):
        return tc.dynamic_int4_quant(xs_dev[i]) if per_channel else tc.dynamic_int4_quant_grouped(xs_dev[i], GROUP)

    held = []   # quantised activations of the running step (allocated on the second stream, read on the main one)

    def step(events=None):
        cur = torch.cuda.current_stream(dev)
        pending = None
        if overlap:
            # the second stream starts a step after the main one has finished the previous step; only then are the
            # previous step's buffers released, so the allocator can hand them out again on that stream at once
            quant_stream.wait_stream(cur)
            held.clear()
            with torch.cuda.stream(quant_stream):
                pending = quantise(0) + (torch.cuda.Event(),)
                pending[2].record(quant_stream)
        for i, (name, K, N) in enumerate(SHAPES):
            lin = layers[i]
            if overlap:
                xp, xsc, ready = pending
                held.append((xp, xsc))
                cur.wait_event(ready)
                if i + 1 < len(SHAPES):
                    with torch.cuda.stream(quant_stream):
                        pending = quantise(i + 1) + (torch.cuda.Event(),)
                        pending[2].record(quant_stream)
            else:
                xp, xsc = quantise(i)
            if events is not None:
                e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
                e0.record()
            if per_channel:
                tc.cutlass_int4_scaled_mm(xp, lin.weight_int4, xsc, lin.weight_scale, outs[i], M, lin.out_features, K)
            else:
                tc.cutlass_int4_fused_grouped_gemm(xp, lin.weight_int4, xsc, lin.weight_scale, outs[i], M,
                                                   lin.out_features, GROUP, K // GROUP)
            if events is not None:
                e1.record()
                events.append((i, e0, e1))

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    ops.check_status()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)  # let nvidia-smi come up; the GPU is idle meanwhile
    barrier()
    events = []
    wall0 = time.time()
    t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(args.steps):
        step(events)
    t1.record()
    barrier()
    # the timed region can be a few tens of ms, shorter than the sampler's period: keep the same
    # load running (untimed) until at least one second of samples exists
    while time.time() - wall0 < 1.0:
        step()
        torch.cuda.synchronize()
    wall1 = time.time()
    sampler.t_begin, sampler.t_end = wall0, wall1
    clocks = sampler.stop() if rank == 0 else None
    if clocks is not None:
        clocks["window"] = "timed steps plus untimed repeats of the same step, %.2f s" % (wall1 - wall0)
    ops.check_status()
    elapsed_ms = t0.elapsed_time(t1)
    if world > 1:
        tt = torch.tensor([elapsed_ms], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        elapsed_ms = tt.item()
    ms_per_step = elapsed_ms / args.steps
    value = ops_per_step / (ms_per_step * 1e-3) / 1e12

    # dominant kernel: the W4A4 GEMM (this rank's launches), averaged per shape over the timed region
    per_shape = {}
    for i, e0, e1 in events:
        per_shape.setdefault(i, []).append(e0.elapsed_time(e1) * 1e-3)
    gemm_s = sum(statistics.mean(v) for v in per_shape.values())
    gemm_ops_rank = ops_per_step / world
    int8_peak = 2.0 * peaks["bf16_tflops"]
    achieved = gemm_ops_rank / gemm_s / 1e12

    # ---- e2e: host buffers through the linear module, copies inside the timed region.  The ranks share one host:
    # each copies M / n rows of the activations from pinned memory and an all-gather over NVLink gives every rank
    # the whole [M, K] (the GEMM itself stays free of collectives); each rank reads back its own output columns.
    assert M % world == 0
    m_loc = M // world
    x_host = [synthetic.activations(M, K, seed=0)[rank * m_loc:(rank + 1) * m_loc].contiguous().pin_memory()
              for _, K, _ in SHAPES]
    o_host = [torch.empty(M, l.out_features, dtype=torch.bfloat16).pin_memory() for l in layers]
    h2d = sum(x.numel() * 2 for x in x_host) * world   # whole job
    d2h = sum(o.numel() * 2 for o in o_host) * world

    copy_in, copy_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    main = torch.cuda.current_stream(dev)

    def e2e_step():
        # host -> device on one stream, the linear on the main stream, device -> host on a third:
        # the three overlap across the four linears of a step
        prev = None
        for i, lin in enumerate(layers):
            with torch.cuda.stream(copy_in):
                xd = x_host[i].to(dev, non_blocking=True)
                if world > 1:
                    full = torch.empty(M, xd.shape[1], dtype=xd.dtype, device=dev)
                    dist.all_gather_into_tensor(full, xd)
                    xd = full
                ready = torch.cuda.Event()
                ready.record(copy_in)
            main.wait_event(ready)
            y = lin(xd)
            xd.record_stream(main)
            done = torch.cuda.Event()
            done.record(main)
            with torch.cuda.stream(copy_out):
                copy_out.wait_event(done)
                o_host[i].copy_(y, non_blocking=True)
            y.record_stream(copy_out)
            prev = y
        torch.cuda.synchronize()

    for _ in range(2):
        e2e_step()
    barrier()
    e2e_steps = max(1, min(args.steps, 5))
    w0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    barrier()
    e2e_s = (time.perf_counter() - w0) / e2e_steps
    if world > 1:
        tt = torch.tensor([e2e_s], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        e2e_s = tt.item()
    e2e_val = ops_per_step / e2e_s / 1e12

    del x_host, o_host
    for lin in layers:
        lin.weight_int4 = None
    del layers, xs_dev, outs
    torch.cuda.empty_cache()
    moe_result = bench_moe(args, world, rank, dev, peaks)
    # the same layer with 4096 tokens per rank (weak scaling), where the exchange is no longer latency-bound
    moe_weak = bench_moe(args, world, rank, dev, peaks, weak=True) if world > 1 else None

    if rank == 0:
        line = {
            "metric": METRIC_CHANNEL if per_channel else METRIC, "value": value, "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "s4*s4->s32, f32 dequant", "data": "synthetic",
            "config": workload_config(M, world, per_channel), "clocks": clocks,
            "e2e": {"value": e2e_val, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h * 1,
                    "ms_per_step": e2e_s * 1e3},
            "gpu_launches": args.steps * 2 * len(SHAPES),   # timed region of `value`: quantise + GEMM per linear
            "roofline": {
                "bound": "tensor", "achieved": achieved, "peak": int8_peak, "unit": "TOPS",
                "frac": achieved / int8_peak,
                # ncu (M=1024 capture, profiles/): DRAM reads of a launch = 1.00 x its operand bytes and the
                # bf16 output is written back after the kernel ends, so a launch moves its algorithmic bytes
                "traffic": sum(gemm_bytes(M, N // world, K) for _, K, N in SHAPES) / len(SHAPES),
                "traffic_unit": "bytes per launch (mean of the 4 shapes), algorithmic; ncu-confirmed at M=1024",
                "kernel": ("w4a4_gemm_kernel (per-channel epilogue, 256x256 tiles on SM pairs)" if per_channel
                           else "w4a4_gemm_kernel (per-group-128 epilogue, 256x256 tiles on SM pairs)") + ", 4 launches per step",
                "peak_source": f"2 x bf16 burst of MEASURED_PEAKS.json ({peaks['source']}); int8 dense = 2 x bf16 on B200",
                "per_shape_us": {SHAPES[i][0]: statistics.mean(v) * 1e6 for i, v in per_shape.items()},
            },
        }
        if world == 1:
            torch.set_num_threads(max(1, os.cpu_count() or 1))
            t, cops = cpu_reference_step(16)
            t, cops = cpu_reference_step(16)
            line["cpu_baseline"] = {
                "value": cops / t / 1e12, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
                "sample": "16 of %d token rows of each of the 4 linears, one pass" % M,
            }
        if world == 1 and not args.no_sweep:
            sweep = bench_sweep(dev, peaks)
            line["sweep"] = sweep
            # the north-star bars of the sweep as scalars inside the roofline object
            big = [r for r in sweep if r["M"] >= 1024]
            line["roofline"]["sweep_min_frac_int8_peak_m1024_up"] = min(r["frac_int8_peak"] for r in big)
            line["roofline"]["sweep_min_frac_hbm_m1"] = min(r["frac_hbm"] for r in sweep if r["M"] == 1)
            line["roofline"]["sweep_min_frac_hbm_m16"] = min(r["frac_hbm"] for r in sweep if r["M"] == 16)
        # the other north-star workloads, smallest objects last so that they survive a truncated log
        if moe_weak is not None:
            line["moe_weak"] = moe_weak
        line["moe"] = moe_result
        if world == 1 and not args.no_extras:
            line["prefill"] = bench_prefill(args, dev)
            line["quant"] = bench_quant(dev, peaks)
            line["roofline"]["quant_group_frac_hbm"] = line["quant"]["group"]["frac"]
            line["roofline"]["quant_row_frac_hbm"] = line["quant"]["row"]["frac"]
            line["roofline"]["prefill_tokens_per_s"] = line["prefill"]["value"]
        line["roofline"]["moe_tokens_per_s"] = moe_result["value"]
        emit(line)
    if world > 1:
        dist.destroy_process_group()


def graph_time(fn_list, iters: int = 3) -> float:
    """Mean device time (s) of one call, timed as a CUDA-graph replay of the whole list so that host
    launch overhead does not count.  The list should cycle over enough distinct operands to exceed L2."""
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        for fn in fn_list[:2]:
            fn()
        side.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            for fn in fn_list:
                fn()
        g.replay()
        side.synchronize()
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        e0.record(side)
        for _ in range(iters):
            g.replay()
        e1.record(side)
        side.synchronize()
    return e0.elapsed_time(e1) * 1e-3 / (iters * len(fn_list))


def bench_sweep(dev, peaks) -> list:
    """BASELINE configs[1] sweep, kernel-only: M in {1,16,128,1024,8192} x the four (K,N) shapes, group-128
    fused GEMM (quantise excluded), and beside it the per-channel GEMM of the same shape.  Operands rotate over enough copies to exceed L2 for the HBM-bound sizes."""
    import int4_native_tc as tc
    from fp8_inference_toolkit_b200 import synthetic

    out_rows = []
    int8_peak = 2.0 * peaks["bf16_tflops"]
    for M in (1, 16, 128, 1024, 8192):
        for name, K, N in SHAPES:
            G = K // GROUP
            w_bytes = N * K // 2
            copies = 1 if M >= 1024 else max(2, min(24, (300 << 20) // w_bytes))
            ws_ = [synthetic.random_packed((G, N, 64), 100 + i, dev) for i in range(copies)]
            wsc = torch.rand(G, N, device=dev) * 0.01
            xp = synthetic.random_packed((G, M, 64), 7, dev)
            xsc = torch.rand(G, M, device=dev) * 0.1
            out = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
            reps = 2 if M >= 1024 else 1
            fns = [(lambda w=w: tc.cutlass_int4_fused_grouped_gemm(xp, w, xsc, wsc, out, M, N, GROUP, G))
                   for _ in range(reps) for w in ws_]
            t = graph_time(fns)
            del ws_, fns
            # the same shape with per-channel scales (row-major operands, one dequant per tile)
            wr_ = [synthetic.random_packed((N, K // 2), 200 + i, dev) for i in range(copies)]
            xr = synthetic.random_packed((M, K // 2), 8, dev)
            sa1, sb1 = xsc[0].contiguous(), wsc[0].contiguous()
            fns = [(lambda w=w: tc.cutlass_int4_scaled_mm(xr, w, sa1, sb1, out, M, N, K))
                   for _ in range(reps) for w in wr_]
            tch = graph_time(fns)
            del wr_, fns
            # W4A8 of the same shape: int8 activations x int4 weights held as int8 (per-token / per-channel scales)
            t8 = None
            if M >= 16:
                w8_ = [torch.randint(-8, 8, (N, K), dtype=torch.int8, device=dev) for _ in range(max(1, copies // 2))]
                x8 = torch.randint(-128, 128, (M, K), dtype=torch.int8, device=dev)
                fns = [(lambda w=w: tc.cutlass_w4a8_scaled_mm(x8, w, sa1, sb1, out, M, N, K)) for _ in range(reps) for w in w8_]
                t8 = graph_time(fns)
                del w8_, fns
            ops_ = 2.0 * M * N * K
            byts = gemm_bytes(M, N, K)
            out_rows.append({"M": M, "shape": name, "K": K, "N": N, "us": t * 1e6, "tops": ops_ / t / 1e12,
                             "gbs": byts / t / 1e9, "frac_int8_peak": ops_ / t / 1e12 / int8_peak,
                             "frac_hbm": byts / t / 1e9 / peaks["hbm_gbs"],
                             "per_channel_us": tch * 1e6, "per_channel_tops": ops_ / tch / 1e12,
                             "per_channel_frac_int8_peak": ops_ / tch / 1e12 / int8_peak,
                             "w4a8_us": None if t8 is None else t8 * 1e6,
                             "w4a8_tops": None if t8 is None else ops_ / t8 / 1e12})
    return out_rows


def bench_moe(args, world, rank, dev, peaks, weak: bool = False, tokens: int = 4096) -> dict:
    """MoE grouped W4A4 layer (BASELINE configs[3]): 128 experts, top-8, 4096 tokens, hidden 2048,
    intermediate 768, group-128; experts and tokens split evenly across ranks, all-to-all dispatch and
    combine.  Timed from (token rows, expert ids, routing weights) to the combined bf16 output.
    Outside the timed region rank 0 checks its rows of the expert-parallel output against the single-GPU layer
    over all tokens and all experts (which the GPU tests pin bit for bit to the CPU oracle)."""
    import torch.distributed as dist

    from fp8_inference_toolkit_b200 import moe, moe_ep, ops, synthetic

    T, H, I, E, k = (tokens * world if weak else tokens), 2048, 768, 128, 8
    t_loc, e_loc = T // world, E // world
    x, logits = synthetic.moe_inputs(T, H, E, k, seed=0)
    ids, w = moe.moe_route(logits.to(dev), k)
    sl = slice(rank * t_loc, (rank + 1) * t_loc)
    x_l, ids_l, w_l = x[sl].to(dev).contiguous(), ids[sl].contiguous(), w[sl].contiguous()

    def rank_weights(r):
        gu, dn = synthetic.moe_weights(e_loc, H, I, seed=10 + r, device=dev)
        return moe.MoEWeights.quantize(gu, dn)

    mw = rank_weights(rank)
    ep = moe_ep.ExpertParallelMoE(mw, E, t_loc, k, H, transport=args.ep_transport) if world > 1 else None

    def layer():
        if world == 1:
            return moe.moe_layer(x_l, ids_l, w_l, mw)
        return ep(x_l, ids_l, w_l)

    for _ in range(5):
        out = layer()
    ops.check_status()
    torch.cuda.synchronize()
    # The layer is a chain of short launches, so it is replayed as a CUDA graph where every launch is one of this
    # library's kernels (one GPU, or the peer transport); with NCCL in the chain it runs eagerly.
    launch = "eager"
    graph = None
    if world == 1 or ep.transport == "peer":
        try:
            if world > 1:
                graph, gout = ep.capture(x_l, ids_l, w_l)
            else:
                side = torch.cuda.Stream(dev)
                with torch.cuda.stream(side):
                    layer()
                    side.synchronize()
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph, stream=side):
                        gout = layer()
        except Exception as exc:   # a launch that cannot be captured here: stay eager (every rank takes the same path)
            graph = None
            launch = "eager (capture failed: %s)" % repr(exc)[:120]
        torch.cuda.synchronize()
    if graph is not None:
        eager_layer = layer

        def layer():  # noqa: F811
            graph.replay()
            return gout
        launch = "CUDA graph replay"
        for _ in range(3):
            out = layer()
        ops.check_status()
        torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    steps = max(args.steps, 10)
    e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        out = layer()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    if world > 1:
        tt = torch.tensor([ms], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms = tt.item()
    ops.check_status()
    ops_layer = T * k * (2 * H * 2 * I + 2 * I * H)
    int8_peak = 2.0 * peaks["bf16_tflops"] * world
    res = {
        "metric": "moe_w4a4_tokens_per_s", "scaling": "weak" if weak else "strong",
        "value": T / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
        "ms_per_layer": ms, "tops": ops_layer / (ms * 1e-3) / 1e12,
        "frac_of_int8_peak": ops_layer / (ms * 1e-3) / 1e12 / int8_peak,
        "config": {"workload": "BASELINE configs[3]: 128 experts, top-8 of softmax(N(0,1) logits), %d tokens, "
                               "hidden 2048, intermediate 768, group-128; %d experts and %d tokens per rank"
                               % (T, e_loc, t_loc),
                   "timed": "sort + dispatch + gather-quantise + gate/up GEMM + SwiGLU-quantise + down GEMM + combine",
                   "launch": launch},
    }
    if world > 1:
        res["transport"] = ep.transport + (" (rows stored straight into the destination rank's buffer over NVLink, device-side "
                                           "flags)" if ep.transport == "peer" else " (two all_to_all_single of fixed-size blocks)")
        if getattr(ep, "peer_error", None):
            res["peer_transport_unavailable"] = ep.peer_error[:200]
        res["stages_us"] = ep.stage_times_us(x_l, ids_l, w_l)
        if ep.overflowed():
            res["note"] = "a dispatch buffer overflowed in this run and the step was redone with exact split sizes"
    else:
        res["roofline"] = moe_roofline(moe, x_l, ids_l, w_l, mw, ms, ops_layer, peaks)
    # ---- parity, outside the timed region (rank 0; the weak case holds world x the tokens and is checked the same way)
    if rank == 0 and world > 1:
        full = [rank_weights(r) for r in range(world)]
        mw_all = moe.MoEWeights(torch.cat([f.gate_up_packed for f in full]), torch.cat([f.gate_up_scale for f in full]),
                                torch.cat([f.down_packed for f in full]), torch.cat([f.down_scale for f in full]), E, H, I)
        ref = moe.moe_layer(x.to(dev), ids, w, mw_all)[sl].float()
        got = out.float()
        denom = torch.maximum(ref.abs(), 1e-3 * ref.abs().max())
        res["parity"] = {"checked_rows": int(ref.shape[0]), "against": "single-GPU layer over all tokens and experts",
                         "max_rel": float(((got - ref).abs() / denom).max()),
                         "cos": float(torch.nn.functional.cosine_similarity(got.flatten(), ref.flatten(), dim=0)),
                         "identical": bool(torch.equal(got, ref))}
        del full, mw_all
    if ep is not None:
        ep.close()
    return res


def moe_roofline(moe, x, ids, w, mw, ms_layer, ops_layer, peaks) -> dict:
    """Single-GPU MoE layer stage by stage (CUDA events around each launch group, mean of 10 passes)."""
    T, k = ids.shape
    names = ["sort", "quant_gather", "gemm_gate_up", "silu_quant", "gemm_down", "combine"]
    acc = {n: 0.0 for n in names}
    reps = 10
    for it in range(reps + 2):
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(7)]
        ev[0].record()
        sp, inv, off = moe.moe_sort_tokens(ids, mw.num_experts)
        ev[1].record()
        ap, asc = moe.moe_quant_gather(x, sp, k)
        ev[2].record()
        P = asc.shape[1]
        h = torch.empty((P, 2 * mw.inter), dtype=torch.bfloat16, device=x.device)
        moe.moe_w4a4_grouped_gemm(ap, asc, mw.gate_up_packed, mw.gate_up_scale, off, h, 2 * mw.inter, mw.hidden // 128,
                                  mw.num_experts)
        ev[3].record()
        hp, hs = moe.moe_silu_mul_quant(h)
        ev[4].record()
        y = torch.empty((P, mw.hidden), dtype=torch.bfloat16, device=x.device)
        moe.moe_w4a4_grouped_gemm(hp, hs, mw.down_packed, mw.down_scale, off, y, mw.hidden, mw.inter // 128, mw.num_experts)
        ev[5].record()
        moe.moe_combine(y, inv, w, T, k)
        ev[6].record()
        torch.cuda.synchronize()
        if it >= 2:
            for i, n in enumerate(names):
                acc[n] += ev[i].elapsed_time(ev[i + 1]) * 1e3 / reps
    gemm_us = acc["gemm_gate_up"] + acc["gemm_down"]
    int8_peak = 2.0 * peaks["bf16_tflops"]
    P = T * k
    H, I = mw.hidden, mw.inter
    # bytes a layer has to move once: token rows in, packed rows + scales between the stages, bf16 GEMM outputs, weights
    byts = (T * H * 2 + P * (H // 2 + 4 * H // 128) * 2 + P * 2 * I * 2 * 2 + P * (I // 2 + 4 * I // 128) * 2
            + P * H * 2 * 2 + T * H * 2 + mw.gate_up_packed.numel() + mw.down_packed.numel())
    return {"bound": "tensor", "achieved": ops_layer / (gemm_us * 1e-6) / 1e12, "peak": int8_peak, "unit": "TOPS",
            "frac": ops_layer / (gemm_us * 1e-6) / 1e12 / int8_peak, "kernel": "w4a4_gemm_kernel (grouped-tile scheduler), 2 launches",
            "layer_frac_of_int8_peak": ops_layer / (ms_layer * 1e-3) / 1e12 / int8_peak,
            "layer_bytes": byts, "layer_frac_of_hbm": byts / (ms_layer * 1e-3) / 1e9 / peaks["hbm_gbs"],
            "stages_us": {n: round(v, 1) for n, v in acc.items()}, "gemm_share": gemm_us / sum(acc.values())}


def bench_quant(dev, peaks, M: int = 16384, K: int = 12288, steps: int = 10) -> dict:
    """BASELINE configs[2] at its largest shape: fused quantise+pack of bf16 [M, K] (1 % outlier channels x20), per-token
    and per-group-128 scales; bytes per launch = 2MK + MK/2 + 4 M G (int4_native_tc/profile_bottleneck.py:121-148).
    Two inputs of 403 MB alternate (larger than L2); CUDA events around every launch."""
    import int4_native_tc as tc
    from fp8_inference_toolkit_b200 import synthetic

    xs = [synthetic.activations(M, K, seed=i, outlier_frac=0.01, device=dev) for i in range(2)]
    fns = {"row": lambda x: tc.dynamic_int4_quant(x), "group": lambda x: tc.dynamic_int4_quant_grouped(x, GROUP),
           "clipped": lambda x: tc.dynamic_int4_quant_clipped_grouped(x, GROUP, 0.95),
           "asymmetric": lambda x: tc.dynamic_int4_quant_asymmetric_clipped_grouped(x, GROUP, 0.95, None)}
    res = {}
    for mode, fn in fns.items():
        for i in range(4):
            fn(xs[i & 1])
        torch.cuda.synchronize()
        evs = []
        for i in range(steps):
            e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
            e0.record(); fn(xs[i & 1]); e1.record()
            evs.append((e0, e1))
        torch.cuda.synchronize()
        us = statistics.mean(a.elapsed_time(b) for a, b in evs) * 1e3
        byts = 2 * M * K + M * K // 2 + 4 * M * (1 if mode == "row" else K // GROUP) * (2 if mode == "asymmetric" else 1)
        res[mode] = {"us": us, "GBs": byts / us / 1e3, "frac": byts / us / 1e3 / peaks["hbm_gbs"], "bytes": byts}
    res["config"] = {"workload": f"BASELINE configs[2]: fused quantise+pack, bf16 [{M},{K}]", "bound": "hbm",
                     "peak_GBs": peaks["hbm_gbs"], "peak_source": f"copy bandwidth of MEASURED_PEAKS.json ({peaks['source']})"}
    del xs
    return res


def bench_prefill(args, dev, steps: int = 2) -> dict:
    """BASELINE configs[4]: Qwen3-8B-architecture prefill (36 layers, batch 32 x 512), all linears W4A4 group-128,
    random-init weights; token ids come from pinned host memory and a slice of the result is read back each step."""
    from fp8_inference_toolkit_b200 import ops
    from fp8_inference_toolkit_b200.qwen3 import Qwen3Config, Qwen3Prefill

    cfg = Qwen3Config(layers=args.layers)
    model = Qwen3Prefill(cfg, dev)
    B, S = args.batch, args.seq
    ids_host = torch.randint(0, cfg.vocab, (B, S), generator=torch.Generator().manual_seed(0)).pin_memory()

    def step():
        y = model(ids_host.to(dev, non_blocking=True))
        return y[:, -1, :8].float().cpu()

    step()
    ops.check_status()
    torch.cuda.synchronize()
    e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    ops.check_status()
    ms = e0.elapsed_time(e1) / steps
    lin_ops = 2 * B * S * cfg.layers * sum(N * K for _, K, N in SHAPES)
    del model
    torch.cuda.empty_cache()
    return {"metric": "qwen3_8b_w4a4_prefill_tokens_per_s", "value": B * S / (ms * 1e-3), "unit": "tokens/s",
            "ms_per_step": ms, "steps": steps, "linear_tops": lin_ops / (ms * 1e-3) / 1e12,
            "config": {"workload": "BASELINE configs[4]: Qwen3-8B-shaped prefill, %d layers, batch %d x %d, W4A4 group-128, "
                                   "bf16 attention" % (cfg.layers, B, S)}}


def run_quant(args) -> None:
    """BASELINE configs[2] alone: fused activation quantise+pack of bf16 [M, K] (1 % outlier channels x20), per-token,
    per-group-128, clipped and asymmetric variants; HBM-bound.  One JSON line."""
    torch.cuda.set_device(0)
    peaks = load_peaks()
    res = bench_quant(torch.device("cuda", 0), peaks, args.m, args.k, max(args.steps, 3))
    tot = sum(res[m]["bytes"] for m in ("row", "group")) / ((res["row"]["us"] + res["group"]["us"]) * 1e-6) / 1e9
    emit({
        "metric": "int4_quant_pack_gbs", "value": tot, "unit": "GB/s", "n_gpus": 1, "steps": max(args.steps, 3),
        "warmup": 4, "ms_per_step": (res["row"]["us"] + res["group"]["us"]) * 1e-3, "higher_is_better": True,
        "dtype": "f32 on bf16 -> s4", "data": "synthetic", "config": res["config"],
        "roofline": {"bound": "hbm", "achieved": res["group"]["GBs"], "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": res["group"]["frac"], "traffic": None, "kernel": "quant_grouped_kernel",
                     "per_kernel": {k: v for k, v in res.items() if k != "config"}},
    })


def run_moe(args) -> None:
    """BASELINE configs[3] on one GPU with --tokens tokens (4096 by default; a small count gives a case for ncu)."""
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    peaks = load_peaks()
    res = bench_moe(args, 1, 0, dev, peaks, tokens=args.tokens)
    emit({"metric": res["metric"], "value": res["value"], "unit": res["unit"], "n_gpus": 1, "steps": max(args.steps, 10),
          "warmup": 5, "ms_per_step": res["ms_per_layer"], "higher_is_better": True, "dtype": "s4*s4->s32, f32 dequant",
          "data": "synthetic", "config": res["config"], "roofline": res["roofline"]})


def run_prefill(args) -> None:
    """BASELINE configs[4]: Qwen3-8B-architecture prefill, all linears W4A4 group-128, random-init weights,
    batch 32 x 512 uniform random token ids, attention in bf16 (torch SDPA); tokens/s end to end."""
    from fp8_inference_toolkit_b200 import ops
    from fp8_inference_toolkit_b200.qwen3 import Qwen3Config, Qwen3Prefill

    torch.cuda.set_device(0)
    cfg = Qwen3Config(layers=args.layers)
    model = Qwen3Prefill(cfg, "cuda")
    B, S = args.batch, args.seq
    g = torch.Generator().manual_seed(0)
    ids_host = torch.randint(0, cfg.vocab, (B, S), generator=g).pin_memory()

    def step():
        ids = ids_host.to("cuda", non_blocking=True)
        y = model(ids)
        return y[:, -1, :8].float().cpu()  # a device->host read of the result

    for _ in range(max(args.warmup, 1)):
        step()
    ops.check_status()
    torch.cuda.synchronize()
    e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    ops.check_status()
    ms = e0.elapsed_time(e1) / args.steps
    lin_ops = 2 * B * S * cfg.layers * sum(N * K for _, K, N in SHAPES)
    emit({
        "metric": "qwen3_8b_w4a4_prefill_tokens_per_s", "value": B * S / (ms * 1e-3), "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": max(args.warmup, 1), "ms_per_step": ms, "higher_is_better": True,
        "dtype": "s4*s4->s32 linears, bf16 attention", "data": "synthetic",
        "config": {"workload": "BASELINE configs[4]: Qwen3-8B-shaped prefill, %d layers, batch %d x %d, W4A4 group-128"
                               % (cfg.layers, B, S)},
        "linear_tops": lin_ops / (ms * 1e-3) / 1e12,
    })


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="linear", choices=["linear", "quant", "prefill", "moe"],
                    help="linear: the headline W4A4 linears (default; its line also carries the other workloads); "
                         "quant: quantise+pack only; prefill: Qwen3-8B-shaped prefill; moe: the MoE layer on one GPU")
    ap.add_argument("--tokens", type=int, default=4096, help="tokens of the MoE layer for --workload moe")
    ap.add_argument("--layers", type=int, default=36)
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--seq", type=int, default=512)
    ap.add_argument("--k", type=int, default=12288, help="row length for --workload quant")
    ap.add_argument("--no-sweep", action="store_true", help="skip the kernel-only M x shape sweep")
    ap.add_argument("--ep-transport", default="auto", choices=["auto", "nccl", "peer"],
                    help="exchange of the expert-parallel MoE layer: NCCL all-to-all of fixed-size blocks, or peer stores")
    ap.add_argument("--no-extras", action="store_true", help="skip the quantise+pack and prefill objects of the default line")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--m", type=int, default=None,
                    help="tokens per step (default 8192; 16384, the largest of configs[2], for --workload quant)")
    ap.add_argument("--scales", default="group", choices=["group", "channel"],
                    help="linear workload: per-group-128 scales (the headline) or per-token / per-channel scales")
    args = ap.parse_args()
    claim_stdout()
    if args.m is None:
        args.m = 16384 if args.workload == "quant" else 8192
    if args.workload == "quant":
        run_quant(args)
    elif args.workload == "prefill":
        run_prefill(args)
    elif args.workload == "moe":
        run_moe(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
