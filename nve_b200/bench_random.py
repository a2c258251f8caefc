"""Synthetic decode stack for measurement: the counterpart of `nve bench-random` in the reference
(src/main.rs:1339-1569, `run_bench_random_gpu`).

Same model-shape table (src/main.rs:1352-1357) plus the 70B shape of the scaling configuration; weights
are drawn ~N(0, 0.02) with the shared counter-based generator and quantised on the device by the library's
Q4 quantizer (bit-identical to the reference's host quantizer), norm weights are 1, RoPE tables follow
src/main.rs:1456-1474 (theta 10000, f32 angles), K/V caches are pre-filled ~N(0,1) up to the context length.
Per-layer routing comes from a seeded score vector: scores ~U[0,1), min-max normalised, threshold at the
median so that the top half of the layers runs W4A16 and the rest W4A8.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch

from . import cuda_kernels as ck
from .decode_graph import StaticDecodeGraph
from .gpu_layer import (GpuInferenceState, GpuKvCache, GpuLayerWeights, GpuW4, RoutingConfig, normalize_importance)


@dataclass(frozen=True)
class ModelShape:
    hidden: int
    ffn: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    num_layers: int


# src/main.rs:1352-1357 (1b, 3b, 8b) and the 70B-class shape used for tensor-parallel scaling.
SHAPES: Dict[str, ModelShape] = {
    "1b": ModelShape(2048, 8192, 32, 8, 64, 16),
    "3b": ModelShape(3072, 8192, 24, 8, 128, 28),
    "8b": ModelShape(4096, 14336, 32, 8, 128, 32),
    "70b": ModelShape(8192, 28672, 64, 8, 128, 80),
}

PROJ_STREAMS = {"q": 1, "k": 2, "v": 3, "o": 4, "gate": 5, "up": 6, "down": 7}


def proj_dims(shape: ModelShape) -> Dict[str, Tuple[int, int]]:
    """(N, K) of the seven projections of one layer."""
    qd, kvd = shape.num_heads * shape.head_dim, shape.num_kv_heads * shape.head_dim
    return {"q": (qd, shape.hidden), "k": (kvd, shape.hidden), "v": (kvd, shape.hidden), "o": (shape.hidden, qd),
            "gate": (shape.ffn, shape.hidden), "up": (shape.ffn, shape.hidden), "down": (shape.hidden, shape.ffn)}


def w4_bytes(n: int, k: int) -> int:
    """Bytes of one matrix in the reference's device format: nibbles + one f32 scale per 32 weights."""
    return n * k // 2 + n * (k // 32) * 4


def layer_weight_bytes(shape: ModelShape) -> int:
    return sum(w4_bytes(n, k) for n, k in proj_dims(shape).values())


def seeded_routing(num_layers: int, seed: int) -> Tuple[List[float], RoutingConfig]:
    """Scores ~U[0,1) from the shared generator (stream 9000), normalised as src/main.rs:891-898; the
    threshold is the (L/2)-th smallest normalised score, so `importance < threshold` picks the lower half."""
    scores = _uniform_scores(num_layers, seed)
    norm = normalize_importance(scores)
    thr = sorted(norm)[num_layers // 2]
    return norm, RoutingConfig(False, float(thr))


def _mix64(z: int) -> int:
    m = (1 << 64) - 1
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & m
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & m
    return z ^ (z >> 31)


def _uniform_scores(n: int, seed: int, stream_id: int = 9000) -> List[float]:
    """Host copy of the generator's uniform draw: (mix64(state + (2i+1)*golden) >> 40) * 2^-24."""
    m = (1 << 64) - 1
    st = _mix64((seed ^ ((stream_id * 0xD6E8FEB86659FD93) & m)) & m)
    out = []
    for i in range(n):
        a = _mix64((st + (2 * i + 1) * 0x9E3779B97F4A7C15) & m)
        out.append(float(a >> 40) * 2.0**-24)
    return out


def rope_tables(head_dim: int, max_seq: int, theta: float, device) -> Tuple[torch.Tensor, torch.Tensor]:
    """src/main.rs:1456-1474: f32 frequencies and angles, tables stored as f16 [max_seq, hd/2]."""
    half = head_dim // 2
    i = torch.arange(half, dtype=torch.float32)
    freqs = 1.0 / torch.pow(torch.tensor(theta, dtype=torch.float32), 2.0 * i / head_dim)
    ang = torch.arange(max_seq, dtype=torch.float32)[:, None] * freqs[None, :]
    return ang.cos().to(torch.float16).to(device), ang.sin().to(torch.float16).to(device)


def make_w4(n: int, k: int, seed: int, stream_id: int, device="cuda", row0: int = 0, col0: int = 0,
            full_k: Optional[int] = None) -> GpuW4:
    """One quantised projection.  (row0, col0, full_k) select a shard of the full [*, full_k] matrix so that
    tensor-parallel ranks hold slices of the same weights a single GPU would hold."""
    full_k = k if full_k is None else full_k
    if col0 == 0 and full_k == k:
        w = ck.fill_normal(n * k, seed, stream_id, first=row0 * k, scale=0.02, device=device).view(n, k)
    else:
        w = torch.empty((n, k), dtype=torch.float32, device=device)
        # generate whole rows of the full matrix in slabs and keep the column slice
        slab = max(1, (64 << 20) // (4 * full_k))
        for r in range(0, n, slab):
            rows = min(slab, n - r)
            full = ck.fill_normal(rows * full_k, seed, stream_id, first=(row0 + r) * full_k, scale=0.02, device=device)
            w[r:r + rows] = full.view(rows, full_k)[:, col0:col0 + k]
    nib, sc = ck.q4_quantize(w)
    return GpuW4(nib, sc, None, n, k)


def build_state(shape: ModelShape, seed: int, context: int, max_seq: Optional[int] = None, device="cuda",
                fused: bool = True, num_layers: Optional[int] = None, fill_kv: bool = True) -> Tuple[GpuInferenceState, List[float]]:
    """Weights, caches and routing of the synthetic stack.  Returns (state, normalised importance scores)."""
    layers = shape.num_layers if num_layers is None else num_layers
    max_seq = context if max_seq is None else max_seq
    dims = proj_dims(shape)
    lw: List[GpuLayerWeights] = []
    for li in range(layers):
        ws = {name: make_w4(n, k, seed, 1000 * (li + 1) + PROJ_STREAMS[name], device) for name, (n, k) in dims.items()}
        ones = torch.ones(shape.hidden, dtype=torch.float16, device=device)
        lw.append(GpuLayerWeights(ws["q"], ws["k"], ws["v"], ws["o"], ws["gate"], ws["up"], ws["down"], ones, ones.clone()))
    kv = GpuKvCache(layers, shape.num_kv_heads, max_seq, shape.head_dim, device)
    if fill_kv and context > 1:
        for li in range(layers):
            n = shape.num_kv_heads * max_seq * shape.head_dim
            ck.fill_normal(n, seed, 500000 + 2 * li, dtype=torch.float16, device=device, out=kv.k[li].view(-1))
            ck.fill_normal(n, seed, 500001 + 2 * li, dtype=torch.float16, device=device, out=kv.v[li].view(-1))
    cos, sin = rope_tables(shape.head_dim, max_seq, 10000.0, device)
    norm, routing = seeded_routing(shape.num_layers, seed)
    state = GpuInferenceState(lw, kv, shape.num_heads, shape.num_kv_heads, shape.head_dim, 1e-5, cos, sin, routing, fused)
    # five launches per layer (SiLU*up and the conversion for the down projection inside the gate/up launch) unless
    # NVE_B200_FUSE_SILU=0 asks for the six-launch schedule; both produce the same bits
    state.fuse_silu = os.environ.get("NVE_B200_FUSE_SILU", "1") != "0"
    return state, norm[:layers]


def build_graph(state: GpuInferenceState, shape: ModelShape, importance: List[float]) -> StaticDecodeGraph:
    g = StaticDecodeGraph(state, shape.hidden, shape.ffn, importance)
    g.capture()
    return g


def decode_bytes_per_token(shape: ModelShape, context: int) -> int:
    """Algorithmic HBM bytes of one decoded token: every packed weight once, the 16-bit K/V prefix once."""
    kv = 2 * shape.num_kv_heads * context * shape.head_dim * 2
    return shape.num_layers * (layer_weight_bytes(shape) + kv)


# ----------------------------------------------------------------------------------------------------------
# Command-line driver for one GEMV group (the analogue of the reference's cuda/bench_main.cu): used for
# per-shape timing and as the small, bounded workload for profiler captures.
#
#   python -m nve_b200.bench_random --model 8b --group gateup --route w4a8 --layers 4 --reps 3 [--time]
# ----------------------------------------------------------------------------------------------------------
def gemv_groups(shape: ModelShape) -> Dict[str, Tuple[List[int], int]]:
    """The four GEMV launches of a decode layer: row counts of the matrices that share one launch, and K."""
    qd, kvd = shape.num_heads * shape.head_dim, shape.num_kv_heads * shape.head_dim
    return {"qkv": ([qd, kvd, kvd], shape.hidden), "o": ([shape.hidden], qd),
            "gateup": ([shape.ffn, shape.ffn], shape.hidden), "down": ([shape.hidden], shape.ffn)}


def _main() -> None:
    import argparse

    ap = argparse.ArgumentParser(description="run one GEMV group of the synthetic decode stack")
    ap.add_argument("--model", default="8b", choices=sorted(SHAPES))
    ap.add_argument("--group", default="gateup", choices=["qkv", "o", "gateup", "down"])
    ap.add_argument("--route", default="w4a8", choices=["w4a8", "w4a16"])
    ap.add_argument("--layers", type=int, default=4, help="distinct weight sets to rotate over (keep > L2 in total)")
    ap.add_argument("--reps", type=int, default=3)
    ap.add_argument("--pdl", type=int, default=1)
    ap.add_argument("--time", action="store_true", help="time the launches with CUDA events inside a captured graph")
    ap.add_argument("--batch", type=int, default=1, help="> 1: the batched W4A16 GEMM with this many rows of X")
    ap.add_argument("--attn-batch", type=int, default=0,
                    help="instead of a GEMV group: the fused attention of this many independent sequences in one launch "
                         "(RoPE + K/V write + attention at --context), rotating over --layers cache sets")
    ap.add_argument("--fused-silu", action="store_true",
                    help="--group gateup: the decode step's own launch (RMSNorm prologue, SiLU*up and the conversion for "
                         "the down projection in the epilogue)")
    ap.add_argument("--persistent", action="store_true",
                    help="run whole decode steps of a --layers deep stack through the one-kernel form instead of one group")
    ap.add_argument("--context", type=int, default=1024)
    ap.add_argument("--trace", action="store_true",
                    help="--persistent: print the per-phase time stamps of CTA 0 (barrier wait / staging / run, us)")
    ap.add_argument("--prefetch", type=int, default=-1, help="--persistent: L2 prefetch distance in items per warp")
    a = ap.parse_args()
    from .decode_graph import CapturedSequence, PersistentDecode

    ck.set_pdl(bool(a.pdl))
    if a.attn_batch > 0:
        shape, b, ctx = SHAPES[a.model], a.attn_batch, a.context
        nh, nkv, hd = shape.num_heads, shape.num_kv_heads, shape.head_dim
        cos, sin = rope_tables(hd, ctx, 10000.0, "cuda")
        kcs = [ck.fill_normal(b * nkv * ctx * hd, 1, 10 + i, dtype=torch.float16).view(b, nkv, ctx, hd) for i in range(a.layers)]
        vcs = [ck.fill_normal(b * nkv * ctx * hd, 1, 50 + i, dtype=torch.float16).view(b, nkv, ctx, hd) for i in range(a.layers)]
        q = ck.fill_normal(b * nh * hd, 1, 1, dtype=torch.float16).view(b, nh * hd)
        k = ck.fill_normal(b * nkv * hd, 1, 2, dtype=torch.float16).view(b, nkv * hd)
        v = ck.fill_normal(b * nkv * hd, 1, 3, dtype=torch.float16).view(b, nkv * hd)
        out = torch.empty_like(q)
        d_pos = torch.full((b,), ctx - 1, dtype=torch.int32, device="cuda")
        d_len = torch.full((b,), ctx, dtype=torch.int32, device="cuda")
        nbytes = 2 * b * nkv * ctx * hd * 2

        def attn_launches(_a=None, _b=None):
            for i in range(a.layers):
                ck.attn_decode_fused_batch(q, k, v, kcs[i], vcs[i], cos, sin, d_pos, d_len, nh, nkv, hd, ctx, hd ** -0.5, out=out)

        torch.cuda.synchronize()
        if not a.time:
            for _ in range(a.reps):
                attn_launches()
            torch.cuda.synchronize()
            print(f"{a.model} attention of {b} sequences at context {ctx}: {a.reps * a.layers} launches of {nbytes / 1e6:.1f} MB")
            return
        seq = CapturedSequence(attn_launches)
        for _ in range(3):
            seq.replay(0, 1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(a.reps):
            seq.replay(0, 1)
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / (a.reps * a.layers)
        seq.destroy()
        print(f"{a.model} attention of {b} sequences at context {ctx}: {us:.2f} us, {nbytes / us / 1e3:.1f} GB/s ({nbytes / 1e6:.1f} MB)")
        return
    if a.persistent:
        import dataclasses

        shape = dataclasses.replace(SHAPES[a.model], num_layers=a.layers)
        state, imp = build_state(shape, 1, a.context, max_seq=a.context)
        if a.prefetch >= 0:
            ck.decode_step_set_prefetch(a.prefetch)
        pers = PersistentDecode(state, shape.hidden, shape.ffn, imp)
        state.set_position(a.context - 1)
        h0 = ck.fill_normal(shape.hidden, 1, 42, dtype=torch.float16).view(1, -1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for i in range(a.reps + 1):
            if i == 1:
                e0.record()
            pers.hidden_buf.copy_(h0)
            pers.step(state.d_pos.data_ptr(), state.d_seqlen.data_ptr())
        e1.record()
        torch.cuda.synchronize()
        nbytes = decode_bytes_per_token(shape, a.context)
        us = e0.elapsed_time(e1) * 1e3 / max(1, a.reps)
        print(f"{a.model} persistent step, {a.layers} layers, context {a.context}: {us:.1f} us/step, "
              f"{nbytes / us / 1e3:.1f} GB/s ({nbytes / 1e6:.1f} MB), error word {pers.error()}")
        if a.trace:
            from . import _ffi

            phases = a.layers * 5
            trace = torch.zeros(2 * phases * 4, dtype=torch.int64, device="cuda")
            _ffi.load().nve_b200_decode_step_set_trace(trace.data_ptr())
            for _ in range(2):
                pers.hidden_buf.copy_(h0)
                pers.step(state.d_pos.data_ptr(), state.d_seqlen.data_ptr())
            torch.cuda.synchronize()
            _ffi.load().nve_b200_decode_step_set_trace(None)
            t = trace.cpu().view(2, phases, 4).numpy()
            names = ["qkv", "attn", "o", "gateup", "down"]
            print("per phase: barrier wait / activation staging / run (us); CTA 0, then the last CTA")
            for cta in range(2):
                for li in range(a.layers):
                    row = []
                    for k in range(5):
                        s4 = t[cta, li * 5 + k]
                        stg = (s4[2] - s4[1]) / 1e3 if s4[2] else 0.0
                        run = (s4[3] - (s4[2] if s4[2] else s4[1])) / 1e3
                        row.append(f"{names[k]} {(s4[1] - s4[0]) / 1e3:.1f}/{stg:.1f}/{run:.1f}")
                    total = (t[cta, li * 5 + 4][3] - t[cta, li * 5][0]) / 1e3
                    print(f"CTA {'0' if cta == 0 else 'last'} layer {li} ({'W4A8' if pers.routes[li] else 'W4A16'}) "
                          f"{total:.1f} us: " + "  ".join(row))
        return
    ns, k = gemv_groups(SHAPES[a.model])[a.group]
    ws = [[make_w4(n, k, 1, 100 * li + j) for j, n in enumerate(ns)] for li in range(a.layers)]
    x = ck.fill_normal(k, 1, 999, dtype=torch.float16)
    xq, xs = ck.quantize_f16_q8(x)
    outs = [torch.empty((1, n), dtype=torch.float16, device="cuda") for n in ns]
    nbytes = sum(w4_bytes(n, k) for n in ns)

    norm_w = torch.ones(k, dtype=torch.float16, device="cuda")
    fq = torch.zeros(ns[0], dtype=torch.int8, device="cuda")
    flo = torch.zeros(ns[0], dtype=torch.uint8, device="cuda")
    fs = torch.zeros(max(1, ns[0] // 32), dtype=torch.float32, device="cuda")
    fcnt = torch.zeros(max(1, ns[0] // 32), dtype=torch.int32, device="cuda")
    xb = yb = scratch = None
    if a.batch > 1:
        xb = ck.fill_normal(a.batch * k, 1, 998, dtype=torch.float16).view(a.batch, k)
        yb = [torch.empty((a.batch, n), dtype=torch.float16, device="cuda") for n in ns]
        nbytes_s = ck.gemm_w4a16_multi_scratch_bytes(a.batch, ns, k)
        scratch = torch.empty(max(nbytes_s, 16), dtype=torch.uint8, device="cuda")

    def launches(_a=None, _b=None):
        for li in range(a.layers):
            if a.batch > 1:  # the matrices of the group in one GEMM launch
                ck.gemm_w4a16_multi(xb, [w.triple() for w in ws[li]], k, outs=yb, scratch=scratch)
                continue
            trip = [w.triple() for w in ws[li]]
            if a.fused_silu and a.group == "gateup":
                q = ({"xq": fq, "xs": fs, "counters": fcnt} if a.route == "w4a8" else
                     {"xlo": flo, "xhi": fq, "xs": fs, "counters": fcnt})
                ck.rmsnorm_gateup_silu(x.view(1, -1), norm_w, 1e-5, None, trip[0], trip[1], k, a.route == "w4a8", mid=outs[0],
                                       quant=q)
                continue
            if a.route == "w4a8":
                ck.matvec_w4a8_multi(xq, xs, trip, k, outs=outs)
            else:
                ck.matvec_w4a16_multi(x, None, trip, k, outs=outs)

    torch.cuda.synchronize()
    if not a.time:
        for _ in range(a.reps):
            launches()
        torch.cuda.synchronize()
        print(f"{a.model} {a.group} {a.route}: {a.reps * a.layers} launches of {nbytes / 1e6:.1f} MB")
        return
    seq = CapturedSequence(launches)
    for _ in range(3):
        seq.replay(0, 1)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(a.reps):
        seq.replay(0, 1)
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (a.reps * a.layers)
    seq.destroy()
    flops = 2.0 * a.batch * sum(ns) * k
    print(f"{a.model} {a.group} {a.route} batch={a.batch} pdl={a.pdl}: {us:.2f} us/group, {nbytes / us / 1e3:.1f} GB/s "
          f"({nbytes / 1e6:.1f} MB), {flops / us / 1e6:.1f} TFLOP/s")


if __name__ == "__main__":
    _main()
