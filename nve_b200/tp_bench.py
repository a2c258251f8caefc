"""Multi-GPU arm of the benchmark: the same decode step, tensor-parallel over the ranks torchrun started.

One line per run with, next to the contract keys: `tp_vs_single_rel_err` (the tensor-parallel hidden state against the
unsharded stack on rank 0, truncated depth), `collective_ab` (the all-reduce fused into the GEMV against plain NCCL
all-reduce, both launched eagerly, with their mutual error) and `config5_70b` (the 70B-shaped stack on the same ranks).
"""
from __future__ import annotations

import gc
import json
import os
import sys

import torch
import torch.distributed as dist

from . import cuda_kernels as ck
from .bench_random import SHAPES, build_state, decode_bytes_per_token, proj_dims, w4_bytes
from .decode_graph import CapturedSequence, StaticDecodeGraph
from .gpu_layer import gpu_layer_forward_decode
from .tp import TpContext, build_tp_state, tp_layer_forward, tp_layer_forward_nccl


def _log(*a):
    print(*a, file=sys.stderr, flush=True)


def _timed(fn, iters: int) -> float:
    """ms per call: barrier + synchronize on both sides, CUDA events on the launching stream, max over ranks."""
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    dist.barrier()
    torch.cuda.synchronize()
    a.record()
    for i in range(iters):
        fn(i)
    b.record()
    torch.cuda.synchronize()
    dist.barrier()
    t = torch.tensor([a.elapsed_time(b) / iters], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _ranks_identical(t: torch.Tensor) -> bool:
    mine = t.view(torch.int16).to(torch.int32)
    ref = mine.clone()
    dist.broadcast(ref, src=0)
    same = torch.tensor([int(torch.equal(mine, ref))], device="cuda")
    dist.all_reduce(same, op=dist.ReduceOp.MIN)
    return bool(same.item())


def _peak(bench_main):
    path = os.path.join(os.path.dirname(os.path.abspath(bench_main.__file__)), "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return float(json.load(open(path))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def measure_stack(model: str, seed: int, context: int, rank: int, world: int, ctx: TpContext, steps: int, warmup: int,
                  sampler_cls=None, local_rank: int = 0) -> dict:
    """Build this rank's shards of `model`, capture the step, time it (resident and end-to-end) and its GEMV launches
    alone.  Everything is freed before returning."""
    shape = SHAPES[model]
    state, importance, _plan = build_tp_state(shape, seed, context, rank, world)
    torch.cuda.synchronize()
    dist.barrier()
    pos = context - 1
    h0 = ck.fill_normal(shape.hidden, seed, 42, dtype=torch.float16).view(1, -1)
    graph = StaticDecodeGraph(state, shape.hidden, shape.ffn // world, importance, allreduce=True)
    graph.capture()
    launches_per_step = graph.launches_per_replay

    def step(_i):
        ck.device_copy(graph.hidden_buf, h0)
        graph.replay_resident(pos)

    for i in range(warmup):
        step(i)
    sampler = sampler_cls(local_rank) if (sampler_cls is not None and rank == 0) else None
    ms_step = _timed(step, steps)
    clocks = sampler.stop() if sampler else None
    finite = bool(torch.isfinite(graph.hidden_buf.float()).all())
    err = ctx.error()
    same = _ranks_identical(graph.hidden_buf)

    host_in = torch.empty((1, shape.hidden), dtype=torch.float16).pin_memory()
    host_in.copy_(h0.cpu())
    host_out = torch.empty((1, shape.hidden), dtype=torch.float16).pin_memory()

    def step_e2e(_i):
        graph.hidden_buf.copy_(host_in, non_blocking=True)
        graph.replay_resident(pos)
        host_out.copy_(graph.hidden_buf, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for i in range(3):
        step_e2e(i)
    e2e_steps = max(10, steps // 4)
    ms_e2e = _timed(step_e2e, e2e_steps)
    graph.destroy()

    # the step's GEMV launches alone (including the fused all-reduce of o_proj / down_proj)
    s, hbuf, routes = graph.s, graph.hidden_buf, graph.routes

    def record(_a, _b):
        eps = state.norm_eps
        for li, w in enumerate(state.layer_weights):
            qkv = [w.q_proj.triple(), w.k_proj.triple(), w.v_proj.triple()]
            gu = [w.gate_proj.triple(), w.up_proj.triple()]
            qo = [s.q.view(1, -1), s.k.view(1, -1), s.v.view(1, -1)]
            if routes[li]:
                ck.rmsnorm_matvec_w4a8_multi(hbuf, w.input_norm, eps, qkv, w.q_proj.k, outs=qo)
                ck.matvec_w4a8_allreduce(s.xq_a, s.xs_a, [w.o_proj.triple()], w.o_proj.k, outs=[hbuf], residuals=[hbuf])
                ck.rmsnorm_matvec_w4a8_multi(hbuf, w.post_attn_norm, eps, gu, w.gate_proj.k, outs=[s.gate, s.up])
                ck.matvec_w4a8_allreduce(s.xq_f, s.xs_f, [w.down_proj.triple()], w.down_proj.k, outs=[hbuf], residuals=[hbuf])
            else:
                ck.rmsnorm_matvec_w4a16_multi(hbuf, w.input_norm, eps, None, qkv, w.q_proj.k, outs=qo)
                ck.matvec_w4a16_allreduce(s.attn, None, [w.o_proj.triple()], w.o_proj.k, outs=[hbuf], residuals=[hbuf])
                ck.rmsnorm_matvec_w4a16_multi(hbuf, w.post_attn_norm, eps, None, gu, w.gate_proj.k, outs=[s.gate, s.up])
                ck.matvec_w4a16_allreduce(s.gate, None, [w.down_proj.triple()], w.down_proj.k, outs=[hbuf], residuals=[hbuf])

    seq = CapturedSequence(record)
    gemv_launches = seq.launches

    def gemv_step(_i):
        ck.device_copy(hbuf, h0)
        seq.replay(pos, context)

    for i in range(5):
        gemv_step(i)
    ms_gemv = _timed(gemv_step, max(20, steps // 4))
    seq.destroy()
    err = max(err, ctx.error())
    dims = proj_dims(shape)
    weight_bytes = shape.num_layers * sum(w4_bytes(n, k) for n, k in dims.values())
    out = {"shape": shape, "ms_step": ms_step, "ms_e2e": ms_e2e, "e2e_steps": e2e_steps, "ms_gemv": ms_gemv,
           "gemv_launches": gemv_launches, "launches_per_step": launches_per_step, "finite": finite, "same": same,
           "err": err, "clocks": clocks, "routes": routes, "weight_bytes": weight_bytes,
           "total_bytes": decode_bytes_per_token(shape, context)}
    del state, graph, seq, s, hbuf
    gc.collect()
    torch.cuda.empty_cache()
    return out


def parity_and_ab(model: str, seed: int, context: int, rank: int, world: int, ctx: TpContext, layers: int = 4) -> dict:
    """On a truncated depth: (1) the tensor-parallel result against the unsharded stack computed on rank 0, (2) the
    fused all-reduce against plain NCCL all-reduce (same shards, eager launches): relative error and tokens/s."""
    shape = SHAPES[model]
    state, imp, _ = build_tp_state(shape, seed, context, rank, world, num_layers=layers, fill_kv=True)
    state_n, _, _ = build_tp_state(shape, seed, context, rank, world, num_layers=layers, fill_kv=True)
    h0 = ck.fill_normal(shape.hidden, seed, 42, dtype=torch.float16).view(1, -1)
    positions = [context - 2, context - 1]

    def run(fwd, st):
        h = h0
        for pos in positions:
            st.set_position(pos)
            for li in range(layers):
                h = fwd(h, li, st, st.d_pos.data_ptr(), st.d_seqlen.data_ptr(), st.routing.use_w4a8(imp[li]))
        return h

    torch.cuda.synchronize()
    dist.barrier()
    h_fused = run(tp_layer_forward, state).clone()
    torch.cuda.synchronize()
    dist.barrier()
    h_nccl = run(tp_layer_forward_nccl, state_n).clone()
    torch.cuda.synchronize()

    def rel(a, b):
        a, b = a.double().view(-1), b.double().view(-1)
        return float((a - b).abs().max() / b.pow(2).mean().sqrt().clamp_min(1e-30))

    res = {"layers": layers, "fused_vs_nccl_rel_err": rel(h_fused, h_nccl), "ranks_bit_identical_fused": _ranks_identical(h_fused)}
    # eager tokens/s of both forms on this truncated stack (launch-bound: an A/B of the collectives, not a headline)
    state.set_position(context - 1)

    def tok(fwd, st):
        def f(_i):
            h = h0
            for li in range(layers):
                h = fwd(h, li, st, st.d_pos.data_ptr(), st.d_seqlen.data_ptr(), st.routing.use_w4a8(imp[li]))
        for i in range(3):
            f(i)
        return _timed(f, 20)

    state_n.set_position(context - 1)
    ms_f, ms_n = tok(tp_layer_forward, state), tok(tp_layer_forward_nccl, state_n)
    res.update({"fused_eager_us_per_layer": ms_f * 1e3 / layers, "nccl_eager_us_per_layer": ms_n * 1e3 / layers})
    # (1) against the unsharded stack on rank 0.  The two paths differ only in the order of the cross-rank f32 sums, but
    # a one-ulp difference in a hidden state flips int8 codes further down, so a free-running comparison measures how
    # chaotic the stack is, not the kernels.  The layer-wise figure therefore feeds both paths the SAME input per
    # layer (the tensor-parallel trajectory; q/k/v are column-parallel, so the K/V caches stay bit-identical too) and
    # takes the worst layer; the free-running figure is reported beside it.
    errs = torch.zeros(2, device="cuda", dtype=torch.float64)
    state_t, _, _ = build_tp_state(shape, seed, context, rank, world, num_layers=layers, fill_kv=True)
    full = imp_full = None
    if rank == 0:
        full, imp_full = build_state(shape, seed, context, num_layers=layers, fill_kv=True)
    h_in, worst = h0, 0.0
    for pos in positions:
        state_t.set_position(pos)
        for li in range(layers):
            h_tp = tp_layer_forward(h_in, li, state_t, state_t.d_pos.data_ptr(), state_t.d_seqlen.data_ptr(),
                                    state_t.routing.use_w4a8(imp[li]))
            if rank == 0:
                h_s = gpu_layer_forward_decode(h_in, li, full, pos, False, imp_full[li])
                worst = max(worst, rel(h_tp, h_s))
            h_in = h_tp
    torch.cuda.synchronize()
    if rank == 0:
        full2, _ = build_state(shape, seed, context, num_layers=layers, fill_kv=True)
        hf = h0
        for pos in positions:
            for li in range(layers):
                hf = gpu_layer_forward_decode(hf, li, full2, pos, False, imp_full[li])
        torch.cuda.synchronize()
        errs[0], errs[1] = worst, rel(h_fused, hf)
        del full, full2
    dist.broadcast(errs, src=0)
    res["tp_vs_single_rel_err"] = float(errs[0].item())
    res["tp_vs_single_free_running_rel_err"] = float(errs[1].item())
    del state_t
    del state, state_n
    gc.collect()
    torch.cuda.empty_cache()
    return res


def run(args, seed: int, model: str, context: int, workload: str) -> None:
    import __main__ as bench_main  # bench.py, the launcher script

    rank = int(os.environ["RANK"])
    world = int(os.environ["WORLD_SIZE"])
    local_rank = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local_rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    pdl = os.environ.get("NVE_B200_PDL", "1") != "0"
    ck.set_pdl(pdl)
    max_rows = max(SHAPES[model].hidden, SHAPES["70b"].hidden)
    ctx = TpContext(rank, world, max_rows=max_rows)
    torch.cuda.synchronize()
    dist.barrier()

    m = measure_stack(model, seed, context, rank, world, ctx, args.steps, args.warmup, bench_main.ClockSampler, local_rank)
    par = parity_and_ab(model, seed, context, rank, world, ctx)
    big = None
    if model == "8b" and not getattr(args, "quick", False):
        b = measure_stack("70b", seed, context, rank, world, ctx, min(args.steps, 100), 5)
        peak, _ = _peak(bench_main)
        big = {"workload": "Llama-3-70B-shaped decode stack, 80 layers, hidden 8192, FFN 28672, GQA 64/8, batch 1, context "
                           f"{context}, tp{world}",
               "tok_s": 1e3 / b["ms_step"], "ms_per_step": b["ms_step"], "e2e_tok_s": 1e3 / b["ms_e2e"],
               "gemv_gbs_per_gpu": b["weight_bytes"] / world / (b["ms_gemv"] * 1e-3) / 1e9,
               "gemv_frac": b["weight_bytes"] / world / (b["ms_gemv"] * 1e-3) / 1e9 / peak,
               "hbm_gbs_whole_step_per_gpu": b["total_bytes"] / world / (b["ms_step"] * 1e-3) / 1e9,
               "ranks_bit_identical": b["same"], "tp_error": b["err"], "output_finite": b["finite"],
               "launches_per_step": b["launches_per_step"]}
    err = max(m["err"], ctx.error())

    if rank == 0:
        shape = m["shape"]
        per_gpu_bytes = m["weight_bytes"] / world
        peak, peak_src = _peak(bench_main)
        achieved = per_gpu_bytes / (m["ms_gemv"] * 1e-3) / 1e9
        config = bench_main.base_config(shape, m["routes"])
        config.update({"activations": "f16", "kv_cache": "f16", "parallelism": f"tp{world}",
                       "collective": "all-reduce fused into the o_proj / down_proj GEMV kernels: 8-byte {value, epoch} "
                                     "peer stores over NVLink, local polling (NCCL carries handles and barriers only)",
                       "l2_policy": f"{m['weight_bytes'] / world / 1e9:.2f} GB of weights streamed per GPU per step "
                                    "(larger than L2 up to tp4 on the 8B shape)",
                       "launches_per_step": m["launches_per_step"], "programmatic_dependent_launch": pdl})
        line = {
            "metric": "decode_tok_per_s", "value": 1e3 / m["ms_step"], "unit": "tok/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": m["ms_step"], "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "int8", "data": "synthetic", "config": config,
            "hbm_gbs_whole_step_per_gpu": m["total_bytes"] / world / (m["ms_step"] * 1e-3) / 1e9,
            "output_finite": m["finite"], "ranks_bit_identical": m["same"], "tp_error": err,
            "tp_vs_single_rel_err": par["tp_vs_single_rel_err"], "collective_ab": par,
            "clocks": m["clocks"],
            "e2e": {"value": 1e3 / m["ms_e2e"], "unit": "tok/s", "h2d_bytes_per_step": shape.hidden * 2,
                    "d2h_bytes_per_step": shape.hidden * 2, "steps": m["e2e_steps"]},
            "gpu_launches": args.steps * m["launches_per_step"],
            "roofline": {"bound": "hbm", "kernel": "gemv_w4_kernel (per-GPU shard, fused all-reduce included)",
                         "achieved": achieved, "peak": peak, "peak_source": peak_src, "unit": "GB/s",
                         "frac": achieved / peak, "launches_per_step": m["gemv_launches"],
                         "bytes_per_launch": per_gpu_bytes / m["gemv_launches"],
                         "us_per_launch": m["ms_gemv"] * 1e3 / m["gemv_launches"], "traffic": None},
            "cpu_baseline": None,
            "config5_70b": big,
        }
        bench_main.emit(line)
    dist.barrier()
    torch.cuda.synchronize()
    dist.barrier()
    ctx.destroy()
    dist.destroy_process_group()
