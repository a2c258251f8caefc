"""Tensor-parallel decode across the GPUs of one box (one process per GPU).

The reference is single-GPU; this is the Megatron-style split the measurement configuration asks for:
q/k/v and gate/up are column-parallel (split over output rows: heads / FFN rows per rank), o_proj and down_proj
are row-parallel (split over K, a multiple of 32 so quantisation blocks never straddle ranks), and the two
row-parallel GEMVs all-reduce their output.  The all-reduce is fused into the GEMV kernel over CUDA-IPC peer
mappings (`nve_b200_matvec_w4a8_allreduce` / `_w4a16_allreduce`); `torch.distributed` is used only to exchange
the 64-byte IPC handles and for barriers.

Activation quantisation commutes with the split: column-parallel inputs are replicated (identical codes on
every rank) and row-parallel inputs are local slices whose 32-wide groups coincide with the unsharded groups,
so int8 codes and per-block integer accumulators equal the single-GPU ones; only the final cross-rank f32 sum
order differs.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch

from . import _ffi
from . import cuda_kernels as ck
from .bench_random import PROJ_STREAMS, ModelShape, make_w4, rope_tables, seeded_routing
from .gpu_layer import GpuInferenceState, GpuKvCache, GpuLayerWeights, _layer_forward_fused


@dataclass(frozen=True)
class ShardPlan:
    """Which slice of every projection a rank holds: name -> (row0, rows, col0, cols, full_k)."""

    rank: int
    world: int
    local_heads: int
    local_kv_heads: int
    slices: Dict[str, Tuple[int, int, int, int, int]]


def plan_shards(shape: ModelShape, rank: int, world: int) -> ShardPlan:
    """Column split of q/k/v/gate/up, row (K) split of o/down.  Raises when the shape does not divide."""
    if shape.num_heads % world or shape.num_kv_heads % world or shape.ffn % world:
        raise ValueError(f"shape does not divide over {world} ranks")
    hd = shape.head_dim
    lh, lkv, lffn = shape.num_heads // world, shape.num_kv_heads // world, shape.ffn // world
    if (lh * hd) % 32 or lffn % 32:
        raise ValueError("K shards must be multiples of the 32-wide quantisation block")
    qd = shape.num_heads * hd
    s = {
        "q": (rank * lh * hd, lh * hd, 0, shape.hidden, shape.hidden),
        "k": (rank * lkv * hd, lkv * hd, 0, shape.hidden, shape.hidden),
        "v": (rank * lkv * hd, lkv * hd, 0, shape.hidden, shape.hidden),
        "o": (0, shape.hidden, rank * lh * hd, lh * hd, qd),
        "gate": (rank * lffn, lffn, 0, shape.hidden, shape.hidden),
        "up": (rank * lffn, lffn, 0, shape.hidden, shape.hidden),
        "down": (0, shape.hidden, rank * lffn, lffn, shape.ffn),
    }
    return ShardPlan(rank, world, lh, lkv, s)


def exchange_handles(local_handle: bytes, world: int) -> bytes:
    """All-gather the ranks' 64-byte IPC handles through torch.distributed (any backend); rank order."""
    import torch.distributed as dist

    gathered: List[Optional[bytes]] = [None] * world
    dist.all_gather_object(gathered, bytes(local_handle))
    for h in gathered:
        if h is None or len(h) != 64:
            raise RuntimeError("handle exchange failed")
    return b"".join(gathered)  # type: ignore[arg-type]


class TpContext:
    """The library's symmetric buffer of this rank, connected to every peer."""

    def __init__(self, rank: int, world: int, max_rows: int):
        lib = _ffi.load()
        handle = (C.c_ubyte * 64)()
        _ffi.check("nve_b200_tp_create", lib.nve_b200_tp_create(rank, world, max_rows, handle))
        all_handles = exchange_handles(bytes(handle), world)
        buf = (C.c_ubyte * (64 * world)).from_buffer_copy(all_handles)
        _ffi.check("nve_b200_tp_connect", lib.nve_b200_tp_connect(buf))
        self.rank, self.world = rank, world

    @staticmethod
    def error(reset: bool = False) -> int:
        return int(_ffi.load().nve_b200_tp_error(int(reset)))

    def destroy(self) -> None:
        """Free this rank's buffer.  Every peer has it mapped and stores into it from inside the all-reduce kernels, so
        call this only after ALL ranks have synchronised their streams and passed a host barrier."""
        _ffi.load().nve_b200_tp_destroy()


def build_tp_state(shape: ModelShape, seed: int, context: int, rank: int, world: int, device="cuda",
                   num_layers: Optional[int] = None, fill_kv: bool = True):
    """This rank's shards of the synthetic stack that `bench_random.build_state` builds on one GPU (same generator
    streams, so the union of the shards is exactly the single-GPU model).  Returns (state, importance, plan)."""
    plan = plan_shards(shape, rank, world)
    layers = shape.num_layers if num_layers is None else num_layers
    lw: List[GpuLayerWeights] = []
    for li in range(layers):
        ws = {}
        for name, (row0, rows, col0, cols, full_k) in plan.slices.items():
            ws[name] = make_w4(rows, cols, seed, 1000 * (li + 1) + PROJ_STREAMS[name], device, row0=row0, col0=col0,
                               full_k=full_k)
        ones = torch.ones(shape.hidden, dtype=torch.float16, device=device)
        lw.append(GpuLayerWeights(ws["q"], ws["k"], ws["v"], ws["o"], ws["gate"], ws["up"], ws["down"], ones, ones.clone()))
    kv = GpuKvCache(layers, plan.local_kv_heads, context, shape.head_dim, device)
    if fill_kv and context > 1:
        per_head = context * shape.head_dim
        for li in range(layers):
            # the slice of the single-GPU cache that belongs to this rank's KV heads
            first = rank * plan.local_kv_heads * per_head
            n = plan.local_kv_heads * per_head
            ck.fill_normal(n, seed, 500000 + 2 * li, first=first, dtype=torch.float16, device=device, out=kv.k[li].view(-1))
            ck.fill_normal(n, seed, 500001 + 2 * li, first=first, dtype=torch.float16, device=device, out=kv.v[li].view(-1))
    cos, sin = rope_tables(shape.head_dim, context, 10000.0, device)
    norm, routing = seeded_routing(shape.num_layers, seed)
    state = GpuInferenceState(lw, kv, plan.local_heads, plan.local_kv_heads, shape.head_dim, 1e-5, cos, sin, routing, True)
    # With the FFN split over the ranks the quantiser in the down prologue handles only ffn / world values, so the
    # five-launch layer (SiLU*up in the gate/up epilogue) saves a whole dependent launch; NVE_B200_FUSE_SILU=0 keeps six.
    state.fuse_silu = os.environ.get("NVE_B200_FUSE_SILU", "1") != "0"
    # the FFN shard is short: converting it in the down prologue beats the count-and-convert tail of the gate/up launch
    # (measured: 1031 vs 997 tok/s at tp4, 963 vs 917 at tp8, equal at tp2)
    state.convert_in_down_prologue = os.environ.get("NVE_B200_CONVERT_IN_PROLOGUE", "1") != "0"
    return state, norm[:layers], plan


def tp_layer_forward(hidden: torch.Tensor, li: int, state: GpuInferenceState, d_pos: int, d_seqlen: int, use_w4a8: bool,
                     out: Optional[torch.Tensor] = None, scratch=None) -> torch.Tensor:
    """One layer on this rank; o_proj and down_proj all-reduce inside their kernels."""
    return _layer_forward_fused(hidden, state.layer_weights[li], state, li, d_pos, d_seqlen, use_w4a8, out=out,
                                scratch=scratch, allreduce=True)


def tp_layer_forward_nccl(hidden: torch.Tensor, li: int, state: GpuInferenceState, d_pos: int, d_seqlen: int,
                          use_w4a8: bool) -> torch.Tensor:
    """The same layer with the NAMED collective: the row-parallel GEMVs write this rank's f32 partial sums and
    `torch.distributed.all_reduce` (NCCL over NVLink) adds them; the residual is then added with the roundings of the
    fused kernel (f16(sum), then f16(residual + that)).  This is the A/B baseline and the parity reference of the
    all-reduce fused into the GEMV; it is not captured in a graph (eager launches + NCCL)."""
    import torch.distributed as dist

    w = state.layer_weights[li]
    nh, nkv, hd = state.num_heads, state.num_kv_heads, state.head_dim
    dev, f16, f32 = hidden.device, torch.float16, torch.float32
    ffn = w.gate_proj.n
    q = torch.empty((nh, hd), dtype=f16, device=dev)
    k = torch.empty((nkv, hd), dtype=f16, device=dev)
    v = torch.empty((nkv, hd), dtype=f16, device=dev)
    attn = torch.empty((1, nh * hd), dtype=f16, device=dev)
    gate = torch.empty((1, ffn), dtype=f16, device=dev)
    up = torch.empty((1, ffn), dtype=f16, device=dev)
    qkv_w = [w.q_proj.triple(), w.k_proj.triple(), w.v_proj.triple()]
    qkv_o = [q.view(1, -1), k.view(1, -1), v.view(1, -1)]
    kc, vc = state.kv_cache.k[li], state.kv_cache.v[li]
    max_seq, eps, scale = state.kv_cache.max_seq, state.norm_eps, float(hd) ** -0.5

    def reduce_add(res: torch.Tensor, part: torch.Tensor) -> torch.Tensor:
        dist.all_reduce(part)
        return (res.float() + part.to(f16).float()).to(f16)

    if use_w4a8:
        xq_a = torch.empty(nh * hd, dtype=torch.int8, device=dev)
        xs_a = torch.empty(nh * hd // 32, dtype=f32, device=dev)
        ck.rmsnorm_matvec_w4a8_multi(hidden, w.input_norm, eps, qkv_w, w.q_proj.k, outs=qkv_o)
        ck.attn_decode_fused(q, k, v, kc, vc, state.rope_cos, state.rope_sin, d_pos, d_seqlen, attn.view(nh, hd), nh, nkv, hd,
                             max_seq, scale, out_q=xq_a, out_scales=xs_a)
        part = ck.matvec_w4a8_multi(xq_a, xs_a, [w.o_proj.triple()], w.o_proj.k, out_dtype=f32)[0]
        h1 = reduce_add(hidden, part)
        ck.rmsnorm_matvec_w4a8_multi(h1, w.post_attn_norm, eps, [w.gate_proj.triple(), w.up_proj.triple()], w.gate_proj.k,
                                     outs=[gate, up])
        xq_f, xs_f, _ = ck.silu_mul_quantize_q8(gate, up)
        part = ck.matvec_w4a8_multi(xq_f, xs_f, [w.down_proj.triple()], w.down_proj.k, out_dtype=f32)[0]
        return reduce_add(h1, part)
    ck.rmsnorm_matvec_w4a16_multi(hidden, w.input_norm, eps, w.q_proj.awq_scales, qkv_w, w.q_proj.k, outs=qkv_o)
    ck.attn_decode_fused(q, k, v, kc, vc, state.rope_cos, state.rope_sin, d_pos, d_seqlen, attn.view(nh, hd), nh, nkv, hd,
                         max_seq, scale)
    part = ck.matvec_w4a16_multi(attn, w.o_proj.awq_scales, [w.o_proj.triple()], w.o_proj.k, out_dtype=f32)[0]
    h1 = reduce_add(hidden, part)
    ck.rmsnorm_matvec_w4a16_multi(h1, w.post_attn_norm, eps, w.gate_proj.awq_scales,
                                  [w.gate_proj.triple(), w.up_proj.triple()], w.gate_proj.k, outs=[gate, up])
    ck.silu_mul_inplace(gate, up)
    part = ck.matvec_w4a16_multi(gate, w.down_proj.awq_scales, [w.down_proj.triple()], w.down_proj.k, out_dtype=f32)[0]
    return reduce_add(h1, part)
