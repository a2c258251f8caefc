#!/usr/bin/env python3
"""Benchmark of the quantized decode path on B200: Llama-3.1-8B-shaped decode stack at batch 1.

    python bench.py --gpus N --steps K --warmup W            # this library (one JSON line on stdout)
    python bench.py --impl reference --steps K --warmup W    # the reference's CPU path on the host cores

A step is one decoded token through all layers (per-layer W4A8 / W4A16 routing from a seeded score vector,
context 1024, 16-bit K/V).  `value` is tokens/s with the hidden state resident on the device; `e2e` is the
same step driven through the public replay call with the input row uploaded from pinned host memory and the
output row downloaded every step.  `roofline` describes the dominant kernel (the W4 GEMV) from a live
CUDA-event measurement of the step's GEMV launches alone; `cpu_baseline` times the same token on the host with
the CPU restatement of the reference (oracle/) on a bounded sample with all host threads.

Besides the contract keys the line carries: `gemv_shapes` (every GEMV launch of the step per shape and route),
`config1` / `config2` (the single 8192x2048 W4A16 GEMV and the Llama-3.2-1B W4A8 layer set), `gemm_batch` (the
batched W4A16 GEMM at batch 1..64), `persistent_step` (the same token through the one-kernel form) and
`lm_head` (tokens/s when the final RMSNorm + lm_head GEMV run on the device too).
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
VOCAB = 128256


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
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50", "-i",
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


# ----------------------------------------------------------------------------- the same token on the host
class CpuStack:
    """The decode stack on the host, computed with the CPU restatement of the reference (oracle/): f32 hidden state,
    RMSNorm, Q4 GEMVs (W4A16-routed layers: the reference's CPU path `matvec_f32` on f32 activations; W4A8-routed
    layers: int8 activation quantiser + integer-dot GEMV), RoPE, f32 attention over an f32 K/V cache, SiLU*up.
    One layer's weights are generated and quantised; every layer holds its own copy of the packed bytes (distinct
    memory, so no layer is served from the host caches), in the form its route reads."""

    def __init__(self, shape, routes, seed: int, context: int):
        import numpy as np

        import oracle
        from nve_b200.bench_random import PROJ_STREAMS, proj_dims

        self.np, self.orc, self.shape, self.routes, self.context = np, oracle, shape, list(routes), context
        self.threads = os.cpu_count() or 1
        oracle.set_threads(self.threads)
        blocks, gpu_form = {}, {}
        for name, (n, k) in proj_dims(shape).items():
            w = oracle.fill_normal(n * k, seed, 1000 + PROJ_STREAMS[name], scale=0.02).reshape(n, k)
            blocks[name] = oracle.quantize_q4(w)
            gpu_form[name] = oracle.extract_for_gpu(blocks[name])
            del w
        self.layers = []
        for use_w4a8 in self.routes:
            if use_w4a8:
                self.layers.append({n: (g[0].copy(), g[1].copy()) for n, g in gpu_form.items()})
            else:
                self.layers.append({n: b.copy() for n, b in blocks.items()})
        nkv, hd = shape.num_kv_heads, shape.head_dim
        k0 = oracle.fill_normal(nkv * context * hd, seed, 500000).reshape(nkv, context, hd)
        v0 = oracle.fill_normal(nkv * context * hd, seed, 500001).reshape(nkv, context, hd)
        self.kc = [k0.copy() for _ in self.routes]
        self.vc = [v0.copy() for _ in self.routes]
        self.ones = np.ones(shape.hidden, np.float32)
        self.cos, self.sin = oracle.rope_tables_f32(hd, context, 10000.0)
        self.bytes = sum(b.nbytes for b in blocks.values()) * len(self.routes)

    def _gemv(self, li: int, name: str, x):
        orc, w = self.orc, self.layers[li][name]
        if self.routes[li]:
            xq, xs = orc.quantize_q8(orc.to_act16(x))
            return orc.w4a8_matvec_mt(xq, xs, w[0], w[1])
        return orc.q4_matvec_mt(w, x)

    def token(self, x, pos: int):
        np, orc, s = self.np, self.orc, self.shape
        nh, nkv, hd = s.num_heads, s.num_kv_heads, s.head_dim
        for li in range(len(self.routes)):
            n1 = orc.rms_norm_f64(x, self.ones, 1e-5)
            q, k, v = self._gemv(li, "q", n1), self._gemv(li, "k", n1), self._gemv(li, "v", n1)
            q = orc.rope_apply(q, nh, hd, self.cos[pos], self.sin[pos])
            k = orc.rope_apply(k, nkv, hd, self.cos[pos], self.sin[pos])
            self.kc[li][:, pos] = k
            self.vc[li][:, pos] = v.reshape(nkv, hd)
            a = orc.attn_decode_f32(q, self.kc[li], self.vc[li], pos + 1, float(hd) ** -0.5).reshape(-1)
            x = x + self._gemv(li, "o", a)
            n2 = orc.rms_norm_f64(x, self.ones, 1e-5)
            g, u = self._gemv(li, "gate", n2), self._gemv(li, "up", n2)
            mid = (g / (1.0 + np.exp(-g)) * u).astype(np.float32)
            x = x + self._gemv(li, "down", mid)
        return x


def cpu_routes(shape):
    from nve_b200.bench_random import seeded_routing

    norm, routing = seeded_routing(shape.num_layers, SEED)
    return [routing.use_w4a8(v) for v in norm]


def cpu_sample_text(stack: CpuStack, tokens: int) -> str:
    s = stack.shape
    return (f"{tokens} whole decoded tokens (all {s.num_layers} layers: RMSNorm, 7 Q4 GEMVs, RoPE, f32 attention over "
            f"context {stack.context}, SiLU*up; {sum(stack.routes)} layers on the int8-activation route, "
            f"{len(stack.routes) - sum(stack.routes)} on the reference's f32 `matvec_f32` route) on {stack.threads} "
            f"host threads, AVX2 inner loops, {stack.bytes / 1e9:.2f} GB of packed weights in distinct memory per layer")


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from nve_b200.bench_random import SHAPES

    import oracle

    shape = SHAPES[MODEL]
    t0 = time.perf_counter()
    stack = CpuStack(shape, cpu_routes(shape), SEED, CONTEXT)
    log(f"[bench] host stack built in {time.perf_counter() - t0:.1f}s")
    x = oracle.fill_normal(shape.hidden, SEED, 42)
    pos = CONTEXT - 1
    t0 = time.perf_counter()
    for _ in range(max(1, args.warmup)):
        stack.token(x, pos)
    per_tok = (time.perf_counter() - t0) / max(1, args.warmup)
    # a bounded sample: as many of the requested steps as fit in about a minute and a half
    steps = max(1, min(args.steps, int(90.0 / max(per_tok, 1e-3))))
    t0 = time.perf_counter()
    for _ in range(steps):
        stack.token(x, pos)
    dt = (time.perf_counter() - t0) / steps
    tok_s = 1.0 / dt
    line = {
        "impl": "reference", "metric": "decode_tok_per_s", "value": tok_s, "unit": "tok/s", "n_gpus": args.gpus,
        "steps": steps, "steps_requested": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": base_config(shape, cpu_routes(shape)),
        "cpu_baseline": {"value": tok_s, "unit": "tok/s", "cores": stack.threads, "kind": "port",
                         "sample": cpu_sample_text(stack, steps)},
        "e2e": {"value": tok_s, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    emit(line)


def workload_name() -> str:
    from nve_b200.bench_random import SHAPES

    s = SHAPES[MODEL]
    family = {"8b": "Llama-3.1-8B", "70b": "Llama-3-70B", "1b": "Llama-3.2-1B", "3b": "Llama-3.2-3B"}[MODEL]
    half = s.num_layers // 2
    return (f"{family}-shaped decode stack, batch 1, {s.num_layers} layers, hidden {s.hidden}, FFN {s.ffn}, "
            f"GQA {s.num_heads}/{s.num_kv_heads}, head_dim {s.head_dim}, context {CONTEXT}, 4-bit group-32 weights "
            f"~N(0,0.02), W4A8/W4A16 routed per layer from seeded scores ({s.num_layers - half}/{half})")


def base_config(shape, routes) -> dict:
    """The keys both arms report, so that their lines describe the same workload."""
    return {"workload": workload_name(), "model_shape": MODEL, "context": CONTEXT, "batch": 1,
            "w4a8_layers": int(sum(routes)), "w4a16_layers": int(len(routes) - sum(routes)),
            "lm_head": "not in the timed step (the reference computes final norm + lm_head on the host)"}


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return float(json.load(open(path))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


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


def time_sequence(torch, record_fn, reps: int = 20, warm: int = 3):
    """Capture `record_fn` into the library's graph, replay it; returns (us per replay, launches per replay)."""
    from nve_b200.decode_graph import CapturedSequence

    seq = CapturedSequence(record_fn)
    try:
        for _ in range(warm):
            seq.replay(CONTEXT - 1, CONTEXT)
        ms = time_events(torch, lambda _i: seq.replay(CONTEXT - 1, CONTEXT), reps)
    finally:
        seq.destroy()
    return ms * 1e3, seq.launches


def gemv_shape_table(torch, ck, state, s, hbuf, tmp, shape, peak):
    """Every GEMV launch of the decode step, per projection group and route, rotating over the 32 layers' weights
    (each replay streams 0.3 - 2.3 GB of distinct weights: larger than L2)."""
    from nve_b200.bench_random import proj_dims, w4_bytes

    dims = proj_dims(shape)
    eps = state.norm_eps
    qv, kv_, vv = s.q.view(1, -1), s.k.view(1, -1), s.v.view(1, -1)
    groups = {"qkv": (("q", "k", "v"), shape.hidden), "o": (("o",), dims["o"][1]),
              "gateup": (("gate", "up"), shape.hidden), "down": (("down",), shape.ffn)}
    out = {}
    for gname, (projs, K) in groups.items():
        n_sum = sum(dims[p][0] for p in projs)
        for route in ("w4a8", "w4a16"):
            def rec(_a, _b, gname=gname, route=route):
                for w in state.layer_weights:
                    if gname == "qkv":
                        mats = [w.q_proj.triple(), w.k_proj.triple(), w.v_proj.triple()]
                        if route == "w4a8":
                            ck.rmsnorm_matvec_w4a8_multi(hbuf, w.input_norm, eps, mats, K, outs=[qv, kv_, vv])
                        else:
                            ck.rmsnorm_matvec_w4a16_multi(hbuf, w.input_norm, eps, None, mats, K, outs=[qv, kv_, vv])
                    elif gname == "gateup":
                        mats = [w.gate_proj.triple(), w.up_proj.triple()]
                        if state.fuse_silu:  # the step's own launch: + SiLU*up + conversion for the down projection
                            q = ({"xq": s.xq_f, "xs": s.xs_f, "counters": s.pq_cnt} if route == "w4a8" else
                                 {"xlo": s.xlo_f, "xhi": s.xq_f, "xs": s.xs_f, "counters": s.pq_cnt})
                            ck.rmsnorm_gateup_silu(hbuf, w.post_attn_norm, eps, None, mats[0], mats[1], K, route == "w4a8",
                                                   mid=s.gate, quant=q)
                        elif route == "w4a8":
                            ck.rmsnorm_matvec_w4a8_multi(hbuf, w.post_attn_norm, eps, mats, K, outs=[s.gate, s.up])
                        else:
                            ck.rmsnorm_matvec_w4a16_multi(hbuf, w.post_attn_norm, eps, None, mats, K, outs=[s.gate, s.up])
                    elif gname == "o":
                        if route == "w4a8":
                            ck.matvec_w4a8_multi(s.xq_a, s.xs_a, [w.o_proj.triple()], K, outs=[tmp], residuals=[hbuf])
                        else:
                            ck.matvec_w4a16_multi(s.attn, None, [w.o_proj.triple()], K, outs=[tmp], residuals=[hbuf])
                    else:
                        if route == "w4a8":
                            ck.matvec_w4a8_multi(s.xq_f, s.xs_f, [w.down_proj.triple()], K, outs=[tmp], residuals=[hbuf])
                        else:
                            ck.matvec_w4a16_planes_multi(s.xlo_f, s.xq_f, s.xs_f, [w.down_proj.triple()], K, outs=[tmp],
                                                         residuals=[hbuf])

            us, launches = time_sequence(torch, rec)
            us /= launches
            if route == "w4a8" and gname in ("o", "down"):
                act = K + K // 8
            elif route == "w4a16" and gname == "down":
                act = 2 * K + K // 8
            else:
                act = 2 * K
            nbytes = w4_bytes(n_sum, K) + act + 2 * n_sum + (2 * n_sum if gname in ("o", "down") else 0)
            gbs = nbytes / us / 1e3
            out[f"{gname}_{route}"] = {"N": n_sum, "K": K, "us": round(us, 3), "gbs": round(gbs, 1),
                                       "frac_measured": round(gbs / peak, 4), "frac_8tbs": round(gbs / 8000.0, 4)}
    return out


def config1_entry(torch, ck, peak):
    """Measurement configuration 1: a single W4A16 GEMV of the Llama-3.2-1B up_proj shape (8192 x 2048), 16 distinct matrices
    rotated (168 MB in total, larger than L2)."""
    from nve_b200.bench_random import make_w4, w4_bytes

    n, k, copies = 8192, 2048, 16
    ws = [make_w4(n, k, SEED, 7000 + i) for i in range(copies)]
    x = ck.fill_normal(k, SEED, 7100, dtype=torch.float16).view(1, -1)
    out = torch.empty((1, n), dtype=torch.float16, device="cuda")

    def rec(_a, _b):
        for w in ws:
            ck.matvec_w4a16_multi(x, None, [w.triple()], k, outs=[out])

    us, launches = time_sequence(torch, rec)
    us /= launches
    nbytes = w4_bytes(n, k) + 2 * k + 2 * n
    gbs = nbytes / us / 1e3
    return {"workload": "single W4A16 GEMV 8192x2048 (Llama-3.2-1B up_proj), f16 activations, f32 block scales",
            "us": round(us, 3), "gbs": round(gbs, 1), "frac_measured": round(gbs / peak, 4),
            "frac_8tbs": round(gbs / 8000.0, 4), "bytes": nbytes}


def config2_entry(torch, ck, peak):
    """Measurement configuration 2: the Llama-3.2-1B layer GEMV set on the W4A8 route, 16 layers (0.61 GB of weights)."""
    from nve_b200.bench_random import SHAPES, build_graph, build_state, layer_weight_bytes
    from nve_b200.gpu_layer import RoutingConfig

    shape = SHAPES["1b"]
    state, imp = build_state(shape, SEED, CONTEXT, max_seq=CONTEXT)
    state.routing = RoutingConfig(False, 2.0)  # every layer below the threshold: W4A8
    graph = build_graph(state, shape, imp)
    s, hbuf = graph.s, graph.hidden_buf
    h0 = ck.fill_normal(shape.hidden, SEED, 42, dtype=torch.float16).view(1, -1)

    def step(_i):
        ck.device_copy(hbuf, h0)
        graph.replay_resident(CONTEXT - 1)

    for i in range(5):
        step(i)
    ms_step = time_events(torch, step, 50)
    graph.destroy()
    eps = state.norm_eps
    qv, kv_, vv = s.q.view(1, -1), s.k.view(1, -1), s.v.view(1, -1)

    def rec(_a, _b):
        for w in state.layer_weights:
            ck.rmsnorm_matvec_w4a8_multi(hbuf, w.input_norm, eps, [w.q_proj.triple(), w.k_proj.triple(), w.v_proj.triple()],
                                         w.q_proj.k, outs=[qv, kv_, vv])
            ck.matvec_w4a8_multi(s.xq_a, s.xs_a, [w.o_proj.triple()], w.o_proj.k, outs=[hbuf], residuals=[hbuf])
            ck.rmsnorm_matvec_w4a8_multi(hbuf, w.post_attn_norm, eps, [w.gate_proj.triple(), w.up_proj.triple()],
                                         w.gate_proj.k, outs=[s.gate, s.up])
            ck.matvec_w4a8_multi(s.xq_f, s.xs_f, [w.down_proj.triple()], w.down_proj.k, outs=[hbuf], residuals=[hbuf])

    ck.device_copy(hbuf, h0)
    us, launches = time_sequence(torch, rec)
    nbytes = layer_weight_bytes(shape) * shape.num_layers
    gbs = nbytes / us / 1e3
    return {"workload": "Llama-3.2-1B W4A8 layer GEMV set (q/k/v, o, gate/up, down), 16 layers, batch 1",
            "gemv_set_us_per_layer": round(us / shape.num_layers, 3), "gbs": round(gbs, 1),
            "frac_measured": round(gbs / peak, 4), "frac_8tbs": round(gbs / 8000.0, 4),
            "stack_tok_s": round(1e3 / ms_step, 1), "launches": launches}


def config5_entry(torch, ck, peak, steps: int):
    """Measurement configuration 5 at one GPU: the Llama-3-70B-shaped stack (42.8 GB of packed weights per token), batch 1."""
    from nve_b200.bench_random import SHAPES, build_graph, build_state, decode_bytes_per_token

    shape = SHAPES["70b"]
    state, imp = build_state(shape, SEED, CONTEXT, max_seq=CONTEXT)
    graph = build_graph(state, shape, imp)
    h0 = ck.fill_normal(shape.hidden, SEED, 42, dtype=torch.float16).view(1, -1)

    def step(_i):
        ck.device_copy(graph.hidden_buf, h0)
        graph.replay_resident(CONTEXT - 1)

    for i in range(3):
        step(i)
    ms = time_events(torch, step, steps)
    finite = bool(torch.isfinite(graph.hidden_buf.float()).all())
    launches = graph.launches_per_replay
    graph.destroy()
    total = decode_bytes_per_token(shape, CONTEXT)
    return {"workload": f"Llama-3-70B-shaped decode stack, 80 layers, hidden 8192, FFN 28672, GQA 64/8, batch 1, context "
                        f"{CONTEXT}, tp1", "tok_s": round(1e3 / ms, 2), "ms_per_step": round(ms, 4),
            "hbm_gbs_whole_step": round(total / (ms * 1e-3) / 1e9, 1), "hbm_frac_whole_step": round(total / (ms * 1e-3) / 1e9 / peak, 4),
            "output_finite": finite, "launches_per_step": launches}


def gemm_batch_table(torch, ck, state, shape, peak):
    """Measurement configuration 4: the batched W4A16 path at batch 1 (GEMV) and 8..64 (tensor-core GEMM: mma.sync at 8, tcgen05 above) on the four 8B
    projection groups, rotating over the 32 layers' weights."""
    from nve_b200.bench_random import proj_dims, w4_bytes

    dims = proj_dims(shape)
    groups = {"qkv": (("q_proj", "k_proj", "v_proj"), shape.hidden), "o": (("o_proj",), dims["o"][1]),
              "gateup": (("gate_proj", "up_proj"), shape.hidden), "down": (("down_proj",), shape.ffn)}
    table = {}
    for m in (1, 8, 16, 32, 64):
        row = {}
        for gname, (attrs, K) in groups.items():
            ns = [getattr(state.layer_weights[0], a).n for a in attrs]
            x = ck.fill_normal(m * K, SEED, 8000 + m, dtype=torch.float16).view(m, K)
            outs = [torch.empty((m, n), dtype=torch.float16, device="cuda") for n in ns]
            scratch = None
            if m > 1:
                scratch = torch.empty(max(16, ck.gemm_w4a16_multi_scratch_bytes(m, ns, K)), dtype=torch.uint8, device="cuda")

            def rec(_a, _b, attrs=attrs, K=K, x=x, outs=outs, scratch=scratch, m=m):
                for w in state.layer_weights:
                    trip = [getattr(w, a).triple() for a in attrs]
                    if m == 1:
                        ck.matvec_w4a16_multi(x, None, trip, K, outs=outs)
                    else:
                        ck.gemm_w4a16_multi(x, trip, K, outs=outs, scratch=scratch)

            us, launches = time_sequence(torch, rec, reps=10)
            calls = len(state.layer_weights)
            us /= calls  # per GEMM call: a call whose CTAs cut tiles is two launches (GEMM + partial-tile reduce)
            nbytes = w4_bytes(sum(ns), K)
            gbs = nbytes / us / 1e3
            row[gname] = {"us": round(us, 2), "gbs": round(gbs, 1), "frac": round(gbs / peak, 4),
                          "tflops": round(2.0 * m * sum(ns) * K / us / 1e6, 2), "launches_per_call": launches // calls}
        table[str(m)] = row
    err = ck.gemm_error()
    return table, err


def prefill_entry(torch, ck, state, shape, lengths=(64, 256, 1024)):
    """A prompt block of S positions through all layers with gpu_layer_forward_prefill: projections through
    matmul_x (the fused tensor-core GEMM in 64-row slices up to 128 rows, dequantisation + dense GEMM above, as the
    reference does for every prompt), one-launch RMSNorm rows / KV rows / causal attention.  Eager launches,
    allocations included: the reference has no graph for prefill either (src/gpu_layer.rs:1086-1160)."""
    from nve_b200.gpu_layer import DENSE_ROWS, gpu_layer_forward_prefill

    layers = len(state.layer_weights)
    res = {}
    for S in lengths:
        x = ck.fill_normal(S * shape.hidden, SEED, 9500, dtype=torch.float16).view(S, shape.hidden)

        def run(_i):
            h = x
            for li in range(layers):
                h = gpu_layer_forward_prefill(h, li, state, 0)
            return h

        out = run(0)
        torch.cuda.synchronize()
        finite = bool(torch.isfinite(out.float()).all())
        ms = time_events(torch, run, 3)
        res[str(S)] = {"ms": round(ms, 3), "prompt_tok_s": round(S / (ms * 1e-3), 1), "output_finite": finite,
                       "projections": "dequantise + dense GEMM" if S > DENSE_ROWS else "fused W4A16 GEMM, 64-row slices"}
    res["workload"] = f"prompt block of S positions through all {layers} layers (positions 0..S-1, 16-bit route)"
    res["gemm_error"] = ck.gemm_error()
    return res


def batched_decode_entries(torch, ck, state, shape, batches=(8, 16, 32, 64)):
    """One decode step of B independent sequences (context CONTEXT each) through all layers with
    gpu_layer_forward_decode_batch: tensor-core GEMM projections, one fused RoPE + K/V write + attention launch for all
    sequences, RMSNorm over rows; recorded once into the library's graph (pre-allocated scratch) and replayed.  Tokens per
    second are summed over the sequences.  The reference has no batched decode (its batch > 1 is prefill only)."""
    from nve_b200.gpu_layer import BatchedDecodeScratch, BatchedKvCache, gpu_layer_forward_decode_batch

    layers = len(state.layer_weights)
    out = {}
    for b in batches:
        kv = BatchedKvCache.zeros(layers, b, shape.num_kv_heads, CONTEXT, shape.head_dim)
        for li in range(layers):
            n = kv.k[li].numel()
            ck.fill_normal(n, SEED, 9600 + 2 * li, dtype=torch.float16, out=kv.k[li].view(-1))
            ck.fill_normal(n, SEED, 9601 + 2 * li, dtype=torch.float16, out=kv.v[li].view(-1))
        x = ck.fill_normal(b * shape.hidden, SEED, 9700, dtype=torch.float16).view(b, shape.hidden)
        d_pos = torch.full((b,), CONTEXT - 1, dtype=torch.int32, device="cuda")
        d_len = torch.full((b,), CONTEXT, dtype=torch.int32, device="cuda")
        scratch = BatchedDecodeScratch.make(state, b, shape.hidden, shape.ffn)
        last = {}

        def rec(_a, _b):
            h, res = x, None
            for li in range(layers):  # the add at the end of a layer rides on the next layer's first launch
                r = gpu_layer_forward_decode_batch(h, li, state, kv, d_pos, d_len, scratch, residual=res, defer_add=li < layers - 1)
                h, res = r if li < layers - 1 else (r, None)
            last["h"] = h

        us, launches = time_sequence(torch, rec, reps=5)
        ms = us * 1e-3
        finite = bool(torch.isfinite(last["h"].float()).all())
        kv_bytes = 2 * b * shape.num_kv_heads * CONTEXT * shape.head_dim * 2 * layers
        out[str(b)] = {"ms_per_step": round(ms, 3), "tok_s": round(b / (ms * 1e-3), 1), "launches_per_step": launches,
                       "output_finite": finite, "kv_bytes_read_per_step": kv_bytes}
        del kv, scratch
        torch.cuda.empty_cache()
    out["gemm_error"] = ck.gemm_error()
    return out


def lm_head_entries(torch, ck, state, shape, importance, h0, pos):
    """The same step with the final RMSNorm + lm_head on the device (the reference leaves them on the host): W4
    lm_head (328 MB per token) and dense f16 lm_head (1051 MB per token)."""
    from nve_b200.bench_random import decode_bytes_per_token, w4_bytes
    from nve_b200.decode_graph import StaticDecodeGraph
    from nve_b200.gpu_layer import GpuW4

    nibs, scs = [], []
    slab = 8016  # rows per generated slab (vocab = 16 slabs)
    for r0 in range(0, VOCAB, slab):
        rows = min(slab, VOCAB - r0)
        w = ck.fill_normal(rows * shape.hidden, SEED, 9000, first=r0 * shape.hidden, scale=0.02).view(rows, shape.hidden)
        nb, sc = ck.q4_quantize(w)
        nibs.append(nb)
        scs.append(sc)
        del w
    lm = GpuW4(torch.cat(nibs), torch.cat(scs), None, VOCAB, shape.hidden)
    del nibs, scs
    fnorm = torch.ones(shape.hidden, dtype=torch.float16, device="cuda")
    out = {}
    base = decode_bytes_per_token(shape, CONTEXT)
    variants = [("w4a16", lm, w4_bytes(VOCAB, shape.hidden))]
    dense = ck.fill_normal(VOCAB * shape.hidden, SEED, 9001, scale=0.02, dtype=torch.float16).view(VOCAB, shape.hidden)
    variants.append(("f16", dense, 2 * VOCAB * shape.hidden))
    for kind, w, nbytes in variants:
        g = StaticDecodeGraph(state, shape.hidden, shape.ffn, importance, lm_head=(w, fnorm, kind))
        g.capture()

        def step(_i, g=g):
            ck.device_copy(g.hidden_buf, h0)
            g.replay_resident(pos)

        for i in range(5):
            step(i)
        ms = time_events(torch, step, 100)
        finite = bool(torch.isfinite(g.logits.float()).all())
        g.destroy()
        out[kind] = {"tok_s": round(1e3 / ms, 1), "ms_per_step": round(ms, 4), "lm_head_bytes": nbytes,
                     "hbm_gbs_whole_step": round((base + nbytes) / (ms * 1e-3) / 1e9, 1), "logits_finite": finite}
    return out


def run_ours(args) -> None:
    import torch

    world = int(os.environ.get("WORLD_SIZE", "1"))
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
    from nve_b200.decode_graph import CapturedSequence, PersistentDecode

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
    peak, peak_src = measured_peak()

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
    # keep the device under the same load until the sampler has a few readings of the clocks under it
    t_hold = time.perf_counter()
    while time.perf_counter() - t_hold < 0.4:
        for i in range(50):
            step_resident(i)
        torch.cuda.synchronize()
    gpu_launches = args.steps * launches_per_step
    clocks = sampler.stop()
    step_out = graph.hidden_buf.clone()
    finite = bool(torch.isfinite(step_out.float()).all())

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
    e2e_steps = max(20, args.steps)
    ms_e2e = time_events(torch, step_e2e, e2e_steps)
    graph.destroy()

    # ---- roofline of the dominant kernel: the step's GEMV launches alone, same arguments, same weights
    s = graph.s
    qv, kv_, vv = s.q.view(1, -1), s.k.view(1, -1), s.v.view(1, -1)
    hbuf = graph.hidden_buf

    def record_gemvs(_d_pos, _d_seqlen, fused_gateup=None):
        fused_gateup = state.fuse_silu if fused_gateup is None else fused_gateup
        eps = state.norm_eps
        for li, w in enumerate(state.layer_weights):
            qkv = [w.q_proj.triple(), w.k_proj.triple(), w.v_proj.triple()]
            gu = [w.gate_proj.triple(), w.up_proj.triple()]
            if routes[li]:
                ck.rmsnorm_matvec_w4a8_multi(hbuf, w.input_norm, eps, qkv, w.q_proj.k, outs=[qv, kv_, vv])
                ck.matvec_w4a8_multi(s.xq_a, s.xs_a, [w.o_proj.triple()], w.o_proj.k, outs=[hbuf], residuals=[hbuf])
                if fused_gateup:  # the step's own gate/up launch: SiLU*up + conversion for down in the epilogue
                    ck.rmsnorm_gateup_silu(hbuf, w.post_attn_norm, eps, None, gu[0], gu[1], w.gate_proj.k, True, mid=s.gate,
                                           quant={"xq": s.xq_f, "xs": s.xs_f, "counters": s.pq_cnt})
                else:
                    ck.rmsnorm_matvec_w4a8_multi(hbuf, w.post_attn_norm, eps, gu, w.gate_proj.k, outs=[s.gate, s.up])
                ck.matvec_w4a8_multi(s.xq_f, s.xs_f, [w.down_proj.triple()], w.down_proj.k, outs=[hbuf], residuals=[hbuf])
            else:
                ck.rmsnorm_matvec_w4a16_multi(hbuf, w.input_norm, eps, None, qkv, w.q_proj.k, outs=[qv, kv_, vv])
                ck.matvec_w4a16_multi(s.attn, None, [w.o_proj.triple()], w.o_proj.k, outs=[hbuf], residuals=[hbuf])
                if fused_gateup:
                    ck.rmsnorm_gateup_silu(hbuf, w.post_attn_norm, eps, None, gu[0], gu[1], w.gate_proj.k, False, mid=s.gate,
                                           quant={"xlo": s.xlo_f, "xhi": s.xq_f, "xs": s.xs_f, "counters": s.pq_cnt})
                else:
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
    ms_plain = None
    if state.fuse_silu:
        # the same four GEMV launches per layer in their plain form (gate/up with 16-bit outputs, no SiLU*up and no
        # conversion in its epilogue: the six-launch schedule), for comparison with earlier figures
        seq = CapturedSequence(lambda a, b: record_gemvs(a, b, False))
        for i in range(5):
            gemv_step(i)
        ms_plain = time_events(torch, gemv_step, max(20, args.steps // 4))
        seq.destroy()
    dims = proj_dims(shape)
    act_bytes = 0
    for li in range(shape.num_layers):
        for ks, ns in ((shape.hidden, dims["q"][0] + 2 * dims["k"][0]), (dims["o"][1], shape.hidden),
                       (shape.hidden, 2 * shape.ffn), (shape.ffn, shape.hidden)):
            act_bytes += (ks + ks // 8 if (routes[li] and ks != shape.hidden) else 2 * ks) + 2 * ns
    gemv_bytes = shape.num_layers * sum(w4_bytes(n, k) for n, k in dims.values()) + act_bytes
    achieved = gemv_bytes / (ms_gemv * 1e-3) / 1e9
    # DRAM bytes per launch from ncu captures (dram__bytes_read.sum + dram__bytes_write.sum of a
    # GEMV launch on a > L2 case): 1.0136 x the algorithmic bytes; every block is touched once, so the traffic of a
    # launch grows with its matrix and the ratio carries over to the average launch of the step.
    traffic_ratio = 1.0136
    roofline = {
        "bound": "hbm", "kernel": "gemv_w4_kernel (W4A8 + W4A16 GEMV launches of one decode step)",
        "achieved": achieved, "peak": peak, "peak_source": peak_src, "unit": "GB/s", "frac": achieved / peak,
        "frac_of_8tbs_nominal": achieved / 8000.0, "launches_per_step": gemv_launches,
        "bytes_per_launch": gemv_bytes / gemv_launches, "us_per_launch": ms_gemv * 1e3 / gemv_launches,
        "traffic": traffic_ratio * gemv_bytes / gemv_launches,
        "traffic_source": "ncu captures of GEMV launches on > L2 cases (W4A8 gate/up, W4A16 gate/up, W4A8 o_proj), "
                          "scaled by algorithmic bytes",
    }
    if ms_plain is not None:
        roofline["kernel"] += "; the gate/up launch also applies SiLU*up and converts the result for the down projection"
        roofline["plain_gemv_launches"] = {
            "what": "the same launches with a plain gate/up GEMV (six-launch schedule)",
            "us_per_launch": ms_plain * 1e3 / gemv_launches, "achieved": gemv_bytes / (ms_plain * 1e-3) / 1e9,
            "frac": gemv_bytes / (ms_plain * 1e-3) / 1e9 / peak}

    extras = {}
    if not args.quick and not args.layers and MODEL == "8b":
        tmp = torch.empty_like(hbuf)
        ck.device_copy(hbuf, h0)
        t0 = time.perf_counter()
        extras["gemv_shapes"] = gemv_shape_table(torch, ck, state, s, hbuf, tmp, shape, peak)
        # ---- the same token with the CUDA-core attention kernel in the graph (the default is the tensor-core one):
        # the A/B of that kernel, and the bit-exact reference of the one-kernel form, whose attention phase shares
        # the CUDA-core kernel's arithmetic
        with ck.attn_decode_kernel(cuda_core=True):
            graph_cc = build_graph(state, shape, importance)

        def step_cc(_i):
            ck.device_copy(graph_cc.hidden_buf, h0)
            graph_cc.replay_resident(pos)

        for i in range(5):
            step_cc(i)
        ms_cc = time_events(torch, step_cc, max(50, args.steps // 4))
        step_out_cc = graph_cc.hidden_buf.clone()
        graph_cc.destroy()
        diff = (step_out.float() - step_out_cc.float()).abs().max().item() / max(1e-30, step_out_cc.float().pow(2).mean().sqrt().item())
        extras["cuda_core_attention_step"] = {"tok_s": round(1e3 / ms_cc, 1), "ms_per_step": round(ms_cc, 4),
                                              "timed_with": "one device copy of the input row per step, like persistent_step",
                                              "default_vs_this_max_abs_over_rms": diff}
        # ---- the same token through the one-kernel form
        pers = PersistentDecode(state, shape.hidden, shape.ffn, importance)
        pers.capture()

        def step_pers(_i):
            ck.device_copy(pers.hidden_buf, h0)
            pers.replay_resident(pos)

        for i in range(5):
            step_pers(i)
        ms_pers = time_events(torch, step_pers, max(50, args.steps // 4))
        same = bool(torch.equal(pers.hidden_buf, step_out_cc))
        extras["persistent_step"] = {"tok_s": round(1e3 / ms_pers, 1), "ms_per_step": round(ms_pers, 4), "launches_per_step": 1,
                                     "bit_identical_to_graph_with_cuda_core_attention": same, "error_word": pers.error()}
        pers.destroy()
        extras["lm_head"] = lm_head_entries(torch, ck, state, shape, importance, h0, pos)
        extras["prefill"] = prefill_entry(torch, ck, state, shape)
        extras["batched_decode"] = batched_decode_entries(torch, ck, state, shape)
        table, gerr = gemm_batch_table(torch, ck, state, shape, peak)
        extras["gemm_batch"] = {"rows": table, "error_word": gerr,
                                "tensor_pipe_pct": {"value": 6.4, "source": "sm__pipe_tensor_cycles_active of the gate/up "
                                                    "pair at batch 16 in an ncu --set full capture of the batched GEMM"}}
        del state, graph, pers
        torch.cuda.empty_cache()
        extras["config1"] = config1_entry(torch, ck, peak)
        extras["config2"] = config2_entry(torch, ck, peak)
        torch.cuda.empty_cache()
        extras["config5_70b"] = config5_entry(torch, ck, peak, steps=30)
        torch.cuda.empty_cache()
        log(f"[bench] extra tables in {time.perf_counter() - t0:.1f}s")

    # ---- CPU baseline on a bounded sample (rank 0, N=1 only): the same token on the host
    cpu = None
    if not args.no_cpu_baseline:
        t0 = time.perf_counter()
        import oracle

        full_shape = SHAPES[MODEL]
        stack = CpuStack(full_shape, cpu_routes(full_shape), SEED, CONTEXT)
        x = oracle.fill_normal(full_shape.hidden, SEED, 42)
        stack.token(x, pos)  # warm-up
        t1 = time.perf_counter()
        toks = 0
        while True:
            stack.token(x, pos)
            toks += 1
            if time.perf_counter() - t1 > 12.0 or toks >= 200:
                break
        dt = (time.perf_counter() - t1) / toks
        cpu = {"value": 1.0 / dt, "unit": "tok/s", "cores": stack.threads, "kind": "port",
               "sample": cpu_sample_text(stack, toks)}
        log(f"[bench] host baseline in {time.perf_counter() - t0:.1f}s")
        del stack

    tok_s = 1e3 / ms_step
    total_bytes = decode_bytes_per_token(shape, CONTEXT)
    config = base_config(shape, routes)
    if args.layers:
        config["workload"] += f" -- TRUNCATED to {args.layers} layers"
    config.update({"activations": "f16 (the reference ABI's activation type)", "kv_cache": "f16", "parallelism": "tp1",
                   "l2_policy": f"inputs larger than L2: {total_bytes / 1e9:.2f} GB streamed per step",
                   "launches_per_step": launches_per_step, "graph": f"one CUDA graph per token, {launches_per_step // shape.num_layers} launches per layer",
                   "programmatic_dependent_launch": pdl})
    line = {
        "metric": "decode_tok_per_s", "value": tok_s, "unit": "tok/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "int8", "data": "synthetic", "config": config,
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
    line.update(extras)
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
    ap.add_argument("--quick", action="store_true", help="headline numbers only (no per-shape / batched / 1B tables)")
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
