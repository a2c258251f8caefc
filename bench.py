#!/usr/bin/env python3
"""Benchmark of the quantized decode path on B200: Llama-3.1-8B-shaped decode stack at batch 1.

    python bench.py --gpus N --steps K --warmup W            # this library (one JSON line on stdout)
    python bench.py --impl reference --steps K --warmup W    # the reference's CPU path on the host cores

A step is one decoded token through all layers (per-layer W4A8 / W4A16 routing from a seeded score vector,
context 1024, 16-bit K/V).  `value` is tokens/s with the hidden state resident on the device; `e2e` is the
same step driven through the public replay call with the input row uploaded from pinned host memory and the
output row downloaded every step.  `roofline` describes the dominant kernel (the W4 GEMV) from a live
CUDA-event measurement of the step's GEMV launches alone; `cpu_baseline` times the reference CPU GEMV path
(restated in oracle/) on a bounded sample with all host threads.
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
sys.path.insert(0, ROOT)

SEED = 20240607
CONTEXT = 1024
MODEL = "8b"


def log(*a):
    print(*a, file=sys.stderr, flush=True)


# ----------------------------------------------------------------------------- clocks
class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.proc = None
        self.gpu = gpu_index
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100", "-i",
                 str(gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, smax, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); smax.append(float(f[2])); power.append(float(f[3]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(smax), "power_w_max": max(power),
                "samples": len(sm), "reasons": sorted(reasons)}


# ----------------------------------------------------------------------------- CPU baseline (oracle port)
def cpu_layer_mats(shape, seed: int):
    """The 7 quantised projections of one layer plus an f32 activation vector each, and the thread count."""
    import oracle
    from nve_b200.bench_random import PROJ_STREAMS, proj_dims

    threads = os.cpu_count() or 1
    oracle.set_threads(threads)
    mats = []
    for name, (n, k) in proj_dims(shape).items():
        w = oracle.fill_normal(n * k, seed, 1000 + PROJ_STREAMS[name], scale=0.02).reshape(n, k)
        mats.append((oracle.quantize_q4(w), oracle.fill_normal(k, seed, 77)))
        del w
    return mats, threads


def cpu_one_layer(mats) -> None:
    import oracle

    for blocks, x in mats:
        oracle.q4_matvec_mt(blocks, x)


def cpu_layer_sample(shape, seed: int, budget_s: float):
    """Time one layer's 7 CPU Q4 GEMVs (the oracle's port of the reference's AVX2 path) for about budget_s seconds:
    (seconds per layer, threads, repetitions)."""
    mats, threads = cpu_layer_mats(shape, seed)
    cpu_one_layer(mats)  # warm-up
    t0 = time.perf_counter()
    reps = 0
    while True:
        cpu_one_layer(mats)
        reps += 1
        if time.perf_counter() - t0 > budget_s or reps >= 200:
            break
    return (time.perf_counter() - t0) / reps, threads, reps


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from nve_b200.bench_random import SHAPES

    shape = SHAPES[MODEL]
    mats, threads = cpu_layer_mats(shape, SEED)
    for _ in range(max(1, args.warmup)):
        cpu_one_layer(mats)
    steps = max(1, args.steps)
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_one_layer(mats)
    dt = (time.perf_counter() - t0) / steps
    tok_s = 1.0 / (dt * shape.num_layers)
    sample = (f"one layer (7 Q4 GEMVs, f32 activations) per step on {threads} threads, AVX2 inner loop; "
              f"tokens/s = 1 / (layer time x {shape.num_layers} layers); attention and norms not included")
    line = {
        "impl": "reference", "metric": "decode_tok_per_s", "value": tok_s, "unit": "tok/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(), "model_shape": MODEL, "context": CONTEXT, "batch": 1},
        "cpu_baseline": {"value": tok_s, "unit": "tok/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": tok_s, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    emit(line)


NCU_TRAFFIC_RATIO = 1.0136  # (73.433 MB read + 0.967 MB written) / 73.400 MB algorithmic


def workload_name() -> str:
    from nve_b200.bench_random import SHAPES

    s = SHAPES[MODEL]
    family = {"8b": "Llama-3.1-8B", "70b": "Llama-3-70B", "1b": "Llama-3.2-1B", "3b": "Llama-3.2-3B"}[MODEL]
    half = s.num_layers // 2
    return (f"{family}-shaped decode stack, batch 1, {s.num_layers} layers, hidden {s.hidden}, FFN {s.ffn}, "
            f"GQA {s.num_heads}/{s.num_kv_heads}, head_dim {s.head_dim}, context {CONTEXT}, 4-bit group-32 weights "
            f"~N(0,0.02), W4A8/W4A16 routed per layer from seeded scores ({s.num_layers - half}/{half})")


# ----------------------------------------------------------------------------- GPU arm
def time_events(torch, fn, iters: int) -> float:
    """Milliseconds per call of fn(), CUDA events on the current stream, synchronised on both sides."""
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    a.record()
    for i in range(iters):
        fn(i)
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters


def run_ours(args) -> None:
    import torch

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the CUDA library is the only compute path)")
    torch.cuda.set_device(local_rank)
    if world > 1:
        from nve_b200 import tp_bench

        tp_bench.run(args, SEED, MODEL, CONTEXT, workload_name())
        return

    from nve_b200 import _ffi
    from nve_b200 import cuda_kernels as ck
    from nve_b200.bench_random import (SHAPES, build_graph, build_state, decode_bytes_per_token, proj_dims, w4_bytes)
    from nve_b200.decode_graph import CapturedSequence

    _ffi.load()
    # programmatic dependent launch: every kernel of the step may start while its predecessor drains
    pdl = os.environ.get("NVE_B200_PDL", "1") != "0"
    ck.set_pdl(pdl)
    shape = SHAPES[MODEL]
    if args.layers:  # profiling aid: a shorter stack of the same layers (not the headline workload)
        import dataclasses

        shape = dataclasses.replace(shape, num_layers=args.layers)
    t_build = time.perf_counter()
    state, importance = build_state(shape, SEED, CONTEXT, max_seq=CONTEXT)
    torch.cuda.synchronize()
    log(f"[bench] built {MODEL} stack in {time.perf_counter() - t_build:.1f}s; "
        f"{torch.cuda.memory_allocated() / 1e9:.2f} GB resident")
    pos = CONTEXT - 1
    h0 = ck.fill_normal(shape.hidden, SEED, 42, dtype=torch.float16).view(1, -1)
    graph = build_graph(state, shape, importance)
    routes = graph.routes
    launches_per_step = graph.launches_per_replay

    # ---- value: hidden state resident on the device
    def step_resident(_i):
        ck.device_copy(graph.hidden_buf, h0)
        graph.replay_resident(pos)

    for i in range(args.warmup):
        step_resident(i)
    torch.cuda.synchronize()
    sampler = ClockSampler(local_rank)
    launches0 = ck.launch_count()
    ms_step = time_events(torch, step_resident, args.steps)
    gpu_launches = args.steps * launches_per_step
    clocks = sampler.stop()
    out_check = graph.hidden_buf.float()
    finite = bool(torch.isfinite(out_check).all())

    # ---- e2e: host row in, host row out, every step
    host_in = torch.empty((1, shape.hidden), dtype=torch.float16).pin_memory()
    host_in.copy_(h0.cpu())
    host_out = torch.empty((1, shape.hidden), dtype=torch.float16).pin_memory()

    def step_e2e(_i):
        graph.hidden_buf.copy_(host_in, non_blocking=True)
        graph.replay_resident(pos)
        host_out.copy_(graph.hidden_buf, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for i in range(max(3, args.warmup // 4)):
        step_e2e(i)
    e2e_steps = max(10, args.steps // 4)
    ms_e2e = time_events(torch, step_e2e, e2e_steps)
    graph.destroy()

    # ---- roofline of the dominant kernel: the step's GEMV launches alone, same arguments, same weights
    s = graph.s
    qv, kv_, vv = s.q.view(1, -1), s.k.view(1, -1), s.v.view(1, -1)
    hbuf = graph.hidden_buf

    def record_gemvs(_d_pos, _d_seqlen):
        eps = state.norm_eps
        for li, w in enumerate(state.layer_weights):
            qkv = [w.q_proj.triple(), w.k_proj.triple(), w.v_proj.triple()]
            gu = [w.gate_proj.triple(), w.up_proj.triple()]
            if routes[li]:
                ck.rmsnorm_matvec_w4a8_multi(hbuf, w.input_norm, eps, qkv, w.q_proj.k, outs=[qv, kv_, vv])
                ck.matvec_w4a8_multi(s.xq_a, s.xs_a, [w.o_proj.triple()], w.o_proj.k, outs=[hbuf], residuals=[hbuf])
                ck.rmsnorm_matvec_w4a8_multi(hbuf, w.post_attn_norm, eps, gu, w.gate_proj.k, outs=[s.gate, s.up])
                ck.matvec_w4a8_multi(s.xq_f, s.xs_f, [w.down_proj.triple()], w.down_proj.k, outs=[hbuf], residuals=[hbuf])
            else:
                ck.rmsnorm_matvec_w4a16_multi(hbuf, w.input_norm, eps, None, qkv, w.q_proj.k, outs=[qv, kv_, vv])
                ck.matvec_w4a16_multi(s.attn, None, [w.o_proj.triple()], w.o_proj.k, outs=[hbuf], residuals=[hbuf])
                ck.rmsnorm_matvec_w4a16_multi(hbuf, w.post_attn_norm, eps, None, gu, w.gate_proj.k, outs=[s.gate, s.up])
                # as in the step: the SiLU kernel has left the fixed-point planes of its result in the scratch buffers
                ck.matvec_w4a16_planes_multi(s.xlo_f, s.xq_f, s.xs_f, [w.down_proj.triple()], w.down_proj.k, outs=[hbuf],
                                             residuals=[hbuf])

    seq = CapturedSequence(record_gemvs)
    gemv_launches = seq.launches

    def gemv_step(_i):
        ck.device_copy(hbuf, h0)
        seq.replay(pos, CONTEXT)

    for i in range(5):
        gemv_step(i)
    ms_gemv = time_events(torch, gemv_step, max(20, args.steps // 4))
    seq.destroy()
    dims = proj_dims(shape)
    act_bytes = 0
    for li in range(shape.num_layers):
        for ks, ns in ((shape.hidden, dims["q"][0] + 2 * dims["k"][0]), (dims["o"][1], shape.hidden),
                       (shape.hidden, 2 * shape.ffn), (shape.ffn, shape.hidden)):
            act_bytes += (ks + ks // 8 if (routes[li] and ks != shape.hidden) else 2 * ks) + 2 * ns
    gemv_bytes = shape.num_layers * sum(w4_bytes(n, k) for n, k in dims.values()) + act_bytes
    achieved = gemv_bytes / (ms_gemv * 1e-3) / 1e9
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        peak, peak_src = float(json.load(open(peaks_path))["hbm_gbs"]), "measured"
    else:
        peak, peak_src = 6650.0, "fallback"
    roofline = {
        "bound": "hbm", "kernel": "gemv_w4_kernel (W4A8 + W4A16 GEMV launches of one decode step)",
        "achieved": achieved, "peak": peak, "peak_source": peak_src, "unit": "GB/s", "frac": achieved / peak,
        "frac_of_8tbs_nominal": achieved / 8000.0, "launches_per_step": gemv_launches,
        "bytes_per_launch": gemv_bytes / gemv_launches, "us_per_launch": ms_gemv * 1e3 / gemv_launches,
        # DRAM bytes per launch: dram__bytes_read.sum + dram__bytes_write.sum of the gate/up launch in
        # profiles/gemv_w4a8_gate_up_8b_ncu.md (74.40 MB against 73.40 MB of packed weights: every block is
        # touched once, so traffic grows with the matrix) scaled to the average launch of the step
        "traffic": NCU_TRAFFIC_RATIO * gemv_bytes / gemv_launches,
        "traffic_source": "ncu capture of the gate/up launch (4-layer case, > L2), scaled by algorithmic bytes",
    }

    # ---- CPU baseline on a bounded sample (rank 0, N=1 only)
    cpu = None
    if not args.no_cpu_baseline:
        t_layer, threads, reps = cpu_layer_sample(shape, SEED, budget_s=12.0)
        cpu = {"value": 1.0 / (t_layer * shape.num_layers), "unit": "tok/s", "cores": threads, "kind": "port",
               "sample": f"one layer's 7 Q4 GEMVs (reference CPU path restated in oracle/, AVX2, {threads} threads), "
                         f"{reps} repetitions; tokens/s = 1/(layer time x {shape.num_layers})"}

    tok_s = 1e3 / ms_step
    total_bytes = decode_bytes_per_token(shape, CONTEXT)
    line = {
        "metric": "decode_tok_per_s", "value": tok_s, "unit": "tok/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": workload_name() + (f" -- TRUNCATED to {args.layers} layers" if args.layers else ""),
                   "model_shape": MODEL, "context": CONTEXT, "batch": 1,
                   "activations": "f16 (the reference ABI's activation type)", "kv_cache": "f16",
                   "w4a8_layers": int(sum(routes)), "w4a16_layers": int(len(routes) - sum(routes)),
                   "parallelism": "tp1", "l2_policy": f"inputs larger than L2: {total_bytes / 1e9:.2f} GB streamed per step",
                   "launches_per_step": launches_per_step, "graph": "one CUDA graph per token",
                   "programmatic_dependent_launch": pdl},
        "hbm_gbs_whole_step": total_bytes / (ms_step * 1e-3) / 1e9,
        "hbm_frac_whole_step": total_bytes / (ms_step * 1e-3) / 1e9 / peak,
        "output_finite": finite,
        "clocks": clocks,
        "e2e": {"value": 1e3 / ms_e2e, "unit": "tok/s", "h2d_bytes_per_step": shape.hidden * 2,
                "d2h_bytes_per_step": shape.hidden * 2, "steps": e2e_steps},
        "gpu_launches": gpu_launches,
        "roofline": roofline,
        "cpu_baseline": cpu,
    }
    assert ck.launch_count() - launches0 >= gpu_launches
    emit(line)


_REAL_STDOUT = None


def emit(line: dict) -> None:
    """Print the one JSON line on the process's original stdout."""
    out = _REAL_STDOUT if _REAL_STDOUT is not None else sys.stdout
    out.write(json.dumps(line) + "\n")
    out.flush()


def main() -> None:
    # Libraries (NCCL, for one) print banners on file descriptor 1; keep stdout for the single JSON line by
    # pointing descriptor 1 at stderr for everything else.
    global _REAL_STDOUT, MODEL
    sys.stdout.flush()
    _REAL_STDOUT = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1500)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--layers", type=int, default=0,
                    help="profiling aid: run only this many layers of the stack (default: all; changes the workload)")
    ap.add_argument("--model", default=MODEL, choices=["1b", "3b", "8b", "70b"],
                    help="shape of the synthetic stack; the default is the configuration the headline metric names")
    args = ap.parse_args()
    MODEL = args.model
    args.warmup = max(3, args.warmup) if args.impl == "ours" else max(1, args.warmup)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
