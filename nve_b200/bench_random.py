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
    return state, norm[:layers]


def build_graph(state: GpuInferenceState, shape: ModelShape, importance: List[float]) -> StaticDecodeGraph:
    g = StaticDecodeGraph(state, shape.hidden, shape.ffn, importance)
    g.capture()
    return g


def decode_bytes_per_token(shape: ModelShape, context: int) -> int:
    """Algorithmic HBM bytes of one decoded token: every packed weight once, the 16-bit K/V prefix once."""
    kv = 2 * shape.num_kv_heads * context * shape.head_dim * 2
    return shape.num_layers * (layer_weight_bytes(shape) + kv)
