"""Multi-GPU arm of the benchmark: the same decode step, tensor-parallel over the ranks torchrun started."""
from __future__ import annotations

import json
import os
import sys
import time

import torch
import torch.distributed as dist

from . import cuda_kernels as ck
from .bench_random import SHAPES, decode_bytes_per_token, proj_dims, w4_bytes
from .decode_graph import CapturedSequence, StaticDecodeGraph
from .tp import TpContext, build_tp_state


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


def run(args, seed: int, model: str, context: int, workload: str) -> None:
    import __main__ as bench_main  # bench.py, the launcher script

    ClockSampler = bench_main.ClockSampler

    rank = int(os.environ["RANK"])
    world = int(os.environ["WORLD_SIZE"])
    local_rank = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local_rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    shape = SHAPES[model]
    pdl = os.environ.get("NVE_B200_PDL", "1") != "0"
    ck.set_pdl(pdl)
    state, importance, plan = build_tp_state(shape, seed, context, rank, world)
    ctx = TpContext(rank, world, max_rows=shape.hidden)
    torch.cuda.synchronize()
    dist.barrier()
    pos = context - 1
    h0 = ck.fill_normal(shape.hidden, seed, 42, dtype=torch.float16).view(1, -1)
    local_ffn = shape.ffn // world
    graph = StaticDecodeGraph(state, shape.hidden, local_ffn, importance, allreduce=True)
    graph.capture()
    launches_per_step = graph.launches_per_replay

    def step(_i):
        ck.device_copy(graph.hidden_buf, h0)
        graph.replay_resident(pos)

    for i in range(args.warmup):
        step(i)
    sampler = ClockSampler(local_rank) if rank == 0 else None
    ms_step = _timed(step, args.steps)
    clocks = sampler.stop() if sampler else None
    finite = bool(torch.isfinite(graph.hidden_buf.float()).all())
    err = ctx.error()

    # every rank must hold the same replicated hidden state, bit for bit
    mine = graph.hidden_buf.view(torch.int16).to(torch.int32)
    ref = mine.clone()
    dist.broadcast(ref, src=0)
    same = torch.tensor([int(torch.equal(mine, ref))], device="cuda")
    dist.all_reduce(same, op=dist.ReduceOp.MIN)

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
    e2e_steps = max(10, args.steps // 4)
    ms_e2e = _timed(step_e2e, e2e_steps)
    graph.destroy()

    # the step's GEMV launches alone (including the fused all-reduce of o_proj / down_proj)
    s = graph.s
    hbuf = graph.hidden_buf
    routes = graph.routes

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
    ms_gemv = _timed(gemv_step, max(20, args.steps // 4))
    seq.destroy()
    err = max(err, ctx.error())

    if rank == 0:
        dims = proj_dims(shape)
        weight_bytes = shape.num_layers * sum(w4_bytes(n, k) for n, k in dims.values())
        per_gpu_bytes = weight_bytes / world
        peaks_path = os.path.join(os.path.dirname(os.path.abspath(bench_main.__file__)), "MEASURED_PEAKS.json")
        if os.path.exists(peaks_path):
            peak, peak_src = float(json.load(open(peaks_path))["hbm_gbs"]), "measured"
        else:
            peak, peak_src = 6650.0, "fallback"
        achieved = per_gpu_bytes / (ms_gemv * 1e-3) / 1e9
        total_bytes = decode_bytes_per_token(shape, context)
        line = {
            "metric": "decode_tok_per_s", "value": 1e3 / ms_step, "unit": "tok/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "int8", "data": "synthetic",
            "config": {"workload": workload, "model_shape": model, "context": context, "batch": 1,
                       "activations": "f16", "kv_cache": "f16", "parallelism": f"tp{world}",
                       "collective": "all-reduce fused into the o_proj / down_proj GEMV kernels: 8-byte {value, epoch} peer stores over NVLink, local polling",
                       "l2_policy": "inputs larger than L2 per GPU only up to tp4: "
                                    f"{weight_bytes / world / 1e9:.2f} GB of weights streamed per GPU per step",
                       "launches_per_step": launches_per_step, "programmatic_dependent_launch": pdl,
                       "w4a8_layers": int(sum(routes)), "w4a16_layers": int(len(routes) - sum(routes))},
            "hbm_gbs_whole_step_per_gpu": total_bytes / world / (ms_step * 1e-3) / 1e9,
            "output_finite": finite, "ranks_bit_identical": bool(same.item()), "tp_error": err,
            "clocks": clocks,
            "e2e": {"value": 1e3 / ms_e2e, "unit": "tok/s", "h2d_bytes_per_step": shape.hidden * 2,
                    "d2h_bytes_per_step": shape.hidden * 2, "steps": e2e_steps},
            "gpu_launches": args.steps * launches_per_step,
            "roofline": {"bound": "hbm", "kernel": "gemv_w4_kernel (per-GPU shard, fused all-reduce included)",
                         "achieved": achieved, "peak": peak, "peak_source": peak_src, "unit": "GB/s",
                         "frac": achieved / peak, "launches_per_step": gemv_launches,
                         "bytes_per_launch": per_gpu_bytes / gemv_launches, "us_per_launch": ms_gemv * 1e3 / gemv_launches,
                         "traffic": None},
            "cpu_baseline": None,
        }
        bench_main.emit(line)
    dist.barrier()
    ctx.destroy()
    dist.destroy_process_group()
