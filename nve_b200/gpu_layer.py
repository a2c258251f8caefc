"""Decode-layer call site: per-layer W4A8 / W4A16 routing and the order of kernel calls.

Mirrors the reference's src/gpu_layer.rs for the quantized decode path only: `GpuW4` (:199-205),
`GpuLayerWeights`, the routing predicate of `gpu_layer_forward_decode` (:1005-1025), the attention
sub-layer `gpu_attn_decode` (:633-775) and the SwiGLU FFN `gpu_ffn` (:914-997).  Everything else in that
file (F16 / dequantised weights, prefill, non-Llama FFN types, biases) is outside this package.

Two schedules compute the same thing:
  * ``fused=False`` issues exactly the reference's sequence of kernels (one launch per reference call);
  * ``fused=True`` uses the fused entry points (RMSNorm inside the q/k/v and gate/up GEMV prologue, RoPE +
    KV write + attention + quantise in one kernel, SiLU*up->quantise, residual add in the GEMV epilogue):
    six launches per layer, or five with ``state.fuse_silu`` (SiLU*up and the conversion for the down projection
    inside the gate/up launch).  All give bit-identical hidden states.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import torch

from . import cuda_kernels as ck

Tensor = torch.Tensor


@dataclass
class GpuW4:
    """src/gpu_layer.rs:199-205: packed nibbles [n, k/2] u8, scales [n, k/32] f32, optional awq [k] f32."""

    nibbles: Tensor
    scales: Tensor
    awq_scales: Optional[Tensor]
    n: int
    k: int

    def triple(self):
        return (self.nibbles, self.scales, self.n)


# Rows of x above which matmul_x materialises the weights in f16 and calls the library GEMM.  The sliced kernel
# reads 0.625 bytes per weight per 64 rows (gate+up of an 8B model: 44 us per slice), the dense route writes and
# reads 2 bytes per weight once plus a compute-bound GEMM: level at about two slices, ahead from three.
DENSE_ROWS = 128


def _matmul_dense(x: Tensor, w: GpuW4, out: Optional[Tensor]) -> Tensor:
    """x [M, K] . W^T through `nve_b200_dequant_w4a16` + a dense library GEMM, as src/gpu_layer.rs:220-239 does for
    every M > 1.  Weights are dequantised to f16 (the reference's type); bf16 activations are converted to f16 with
    saturation, like the pre-pass of the fused GEMM, and the result is rounded once to x's type."""
    wf = ck.dequant_w4a16_any(w.nibbles, w.scales, None, w.n, w.k, out_dtype=torch.float16)
    xf = x if x.dtype == torch.float16 else x.float().clamp_(-65504.0, 65504.0).to(torch.float16)
    if out is not None and out.dtype == torch.float16 and out.is_contiguous():
        return torch.matmul(xf, wf.t(), out=out)
    y = torch.matmul(xf, wf.t())
    if out is None:
        return y if y.dtype == x.dtype else y.to(x.dtype)
    out.copy_(y)
    return out


def matmul_x(x: Tensor, w: GpuW4, scratch: Optional[Tensor] = None, out: Optional[Tensor] = None) -> Tensor:
    """`GpuWeight::matmul_x` for W4 weights (src/gpu_layer.rs:220-239): x [M, K] -> [M, N].

    The reference sends M == 1 to `fused_matvec_w4a16` and M > 1 through `dequant_w4a16` + a dense matmul (the whole
    matrix materialised in f16, 4.6 bytes of traffic per weight).  Here M > 1 goes to the tensor-core GEMM that reads the
    packed weights once per slice of up to 64 rows of x; above DENSE_ROWS rows, where the product is bound by
    arithmetic and re-reading the packed weights for every slice costs more than materialising them once, it takes
    the reference's own route (`_matmul_dense`).  The activation multiplier `awq_scales`, which the GEMM has no
    argument for, is applied to x first as the GEMV does per element."""
    if x.dim() != 2 or x.shape[1] != w.k:
        raise ValueError(f"x must be [M, {w.k}]")
    m = x.shape[0]
    if m > DENSE_ROWS:
        if w.awq_scales is not None:
            x = (x.float() * w.awq_scales.view(1, -1)).to(x.dtype)
        return _matmul_dense(x, w, out)
    if m == 1 and out is None:
        return ck.fused_matvec_w4a16(x, w.nibbles, w.scales, w.awq_scales, w.n, w.k)
    if m == 1:
        return ck.matvec_w4a16_multi(x, w.awq_scales, [w.triple()], w.k, outs=[out])[0]
    if w.awq_scales is not None:
        x = (x.float() * w.awq_scales.view(1, -1)).to(x.dtype)
    out = torch.empty((m, w.n), dtype=x.dtype, device=x.device) if out is None else out
    step = 64
    if scratch is None:
        nbytes = ck.gemm_w4a16_scratch_bytes(min(m, step), w.n, w.k)
        scratch = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=x.device)
    for r0 in range(0, m, step):
        rows = min(step, m - r0)
        ck.gemm_w4a16(x[r0:r0 + rows], w.nibbles, w.scales, w.n, w.k, out=out[r0:r0 + rows], scratch=scratch)
    return out


def matmul_x_multi(x: Tensor, ws: Sequence[GpuW4], scratch: Optional[Tensor] = None,
                   outs: Optional[Sequence[Tensor]] = None) -> List[Tensor]:
    """matmul_x for several projections of the same x (q/k/v, gate/up) in one GEMM launch per 64-row slice: their
    tiles share the grid, so narrow projections do not run as few-CTA kernels.  M == 1, M > DENSE_ROWS and weights
    with an activation multiplier go through matmul_x one by one."""
    m, k = x.shape
    if m == 1 or m > DENSE_ROWS or any(w.awq_scales is not None for w in ws):
        return [matmul_x(x, w, scratch, None if outs is None else outs[i]) for i, w in enumerate(ws)]
    outs = [torch.empty((m, w.n), dtype=x.dtype, device=x.device) for w in ws] if outs is None else list(outs)
    step = 64
    ns = [w.n for w in ws]
    if scratch is None:
        scratch = torch.empty(max(16, ck.gemm_w4a16_multi_scratch_bytes(min(m, step), ns, k)), dtype=torch.uint8,
                              device=x.device)
    trip = [w.triple() for w in ws]
    for r0 in range(0, m, step):
        rows = min(step, m - r0)
        ck.gemm_w4a16_multi(x[r0:r0 + rows], trip, k, outs=[o[r0:r0 + rows] for o in outs], scratch=scratch)
    return outs


@dataclass
class GpuLayerWeights:
    """The W4 subset of src/gpu_layer.rs GpuLayerWeights (Llama-style block, no biases)."""

    q_proj: GpuW4
    k_proj: GpuW4
    v_proj: GpuW4
    o_proj: GpuW4
    gate_proj: GpuW4
    up_proj: GpuW4
    down_proj: GpuW4
    input_norm: Tensor
    post_attn_norm: Tensor


@dataclass
class RoutingConfig:
    """Precision routing inputs of src/gpu_layer.rs:1017-1025, read once instead of per call."""

    no_w4a8: bool = False
    threshold: float = 0.7

    @staticmethod
    def from_env(env=os.environ) -> "RoutingConfig":
        no = "NVE_NO_W4A8" in env
        try:
            thr = float(env.get("NVE_W4A8_THRESHOLD", "0.7"))
        except ValueError:
            thr = 0.7  # the reference falls back to the default when the value does not parse
        return RoutingConfig(no, thr)

    def use_w4a8(self, layer_importance: float) -> bool:
        """use_w4a8 = !NVE_NO_W4A8 && importance < threshold (strict)."""
        if self.no_w4a8:
            return False
        return layer_importance < self.threshold


def normalize_importance(scores: Sequence[float]) -> List[float]:
    """src/main.rs:891-898: min-max normalisation to [0,1]; all 0.5 when the range is <= 1e-9."""
    mn, mx = min(scores), max(scores)
    rng = mx - mn
    if rng > 1e-9:
        return [(s - mn) / rng for s in scores]
    return [0.5] * len(scores)


class GpuKvCache:
    """Static per-layer K/V buffers [nkv, max_seq, hd] (the layout of src/decode_graph.rs:183-184).

    The reference's eager path grows its cache with Tensor::cat on every token (src/gpu_layer.rs:468-483);
    here both the eager and the captured path write into pre-allocated buffers.
    """

    def __init__(self, num_layers: int, num_kv_heads: int, max_seq: int, head_dim: int, device, dtype=torch.float16):
        self.max_seq = max_seq
        self.k = [torch.zeros((num_kv_heads, max_seq, head_dim), dtype=dtype, device=device) for _ in range(num_layers)]
        self.v = [torch.zeros((num_kv_heads, max_seq, head_dim), dtype=dtype, device=device) for _ in range(num_layers)]

    def reset(self) -> None:
        pass  # positions are overwritten; the valid length travels with every call


@dataclass
class GpuInferenceState:
    """The fields of src/gpu_layer.rs GpuInferenceState that the quantized decode path reads."""

    layer_weights: List[GpuLayerWeights]
    kv_cache: GpuKvCache
    num_heads: int
    num_kv_heads: int
    head_dim: int
    norm_eps: float
    rope_cos: Tensor  # [max_seq, hd/2] f16
    rope_sin: Tensor
    routing: RoutingConfig = field(default_factory=RoutingConfig)
    fused: bool = True
    # fused schedule only: SiLU*up in the gate/up epilogue, which also converts the result for the down projection
    # (five launches per layer instead of six; same bits)
    fuse_silu: bool = False
    # with fuse_silu: where SiLU*up is converted for the down projection -- False: by the gate/up CTA that completes a
    # 32-wide group (best at one GPU, where every down CTA would otherwise convert the whole FFN vector itself);
    # True: in the prologue of the down GEMV (best under tensor parallelism, where the FFN shard is short and the
    # fence + count + convert tail of the gate/up launch costs more than it saves)
    convert_in_down_prologue: bool = False
    # device scalars for position / valid length of the eager path
    d_pos: Optional[Tensor] = None
    d_seqlen: Optional[Tensor] = None

    def set_position(self, pos: int) -> None:
        if self.d_pos is None:
            dev = self.rope_cos.device
            self.d_pos = torch.zeros(1, dtype=torch.int32, device=dev)
            self.d_seqlen = torch.zeros(1, dtype=torch.int32, device=dev)
        self.d_pos.fill_(pos)
        self.d_seqlen.fill_(min(pos + 1, self.kv_cache.max_seq))


def gpu_attn_decode(normed_or_q8, w: GpuLayerWeights, state: GpuInferenceState, layer_idx: int, d_pos: int,
                    d_seqlen: int, use_w4a8: bool, residual: Optional[Tensor] = None) -> Tensor:
    """src/gpu_layer.rs:633-743 for W4 weights.  `normed_or_q8` is the normed f16 activations (W4A16 route,
    or W4A8 unfused) or an (xq, scales) pair already quantised by the fused prologue.  Returns the o_proj
    output [1, hidden]; with `residual` the residual add is fused into the o_proj epilogue."""
    nh, nkv, hd = state.num_heads, state.num_kv_heads, state.head_dim
    fused = state.fused
    if use_w4a8:
        if isinstance(normed_or_q8, tuple):
            xq, xs = normed_or_q8
        else:
            xq, xs = ck.quantize_f16_q8(normed_or_q8)  # :658
        if fused:
            q, k, v = ck.matvec_w4a8_multi(xq, xs, [w.q_proj.triple(), w.k_proj.triple(), w.v_proj.triple()], w.q_proj.k)
        else:  # :659-661
            q = ck.matvec_w4a8(xq, xs, w.q_proj.nibbles, w.q_proj.scales, w.q_proj.n, w.q_proj.k)
            k = ck.matvec_w4a8(xq, xs, w.k_proj.nibbles, w.k_proj.scales, w.k_proj.n, w.k_proj.k)
            v = ck.matvec_w4a8(xq, xs, w.v_proj.nibbles, w.v_proj.scales, w.v_proj.n, w.v_proj.k)
    else:  # :665-672
        q, k, v = ck.fused_qkv_matvec_w4a16(
            normed_or_q8,
            w.q_proj.nibbles, w.q_proj.scales, w.q_proj.awq_scales, w.q_proj.n,
            w.k_proj.nibbles, w.k_proj.scales, w.k_proj.awq_scales, w.k_proj.n,
            w.v_proj.nibbles, w.v_proj.scales, w.v_proj.awq_scales, w.v_proj.n,
            w.q_proj.k)
    q = q.view(nh, hd)
    k = k.view(nkv, hd)
    v = v.view(nkv, hd)
    ck.rope_decode_dyn_inplace(q, k, state.rope_cos, state.rope_sin, nh, nkv, hd, d_pos)  # :697-711
    kc, vc = state.kv_cache.k[layer_idx], state.kv_cache.v[layer_idx]
    ck.kv_cache_write(k, kc, v, vc, d_pos, nkv, hd, state.kv_cache.max_seq)  # :714
    attn = torch.empty((nh, hd), dtype=torch.float16, device=q.device)
    ck.flash_decode_dyn_into(q, kc, vc, attn, nh, nkv, d_seqlen, hd, float(hd) ** -0.5, state.kv_cache.max_seq)  # :723
    attn = attn.view(1, nh * hd)
    wo = w.o_proj
    if use_w4a8:  # :737-741
        xq2, xs2 = ck.quantize_f16_q8(attn)
        if fused and residual is not None:
            return ck.matvec_w4a8_multi(xq2, xs2, [wo.triple()], wo.k, residuals=[residual])[0]
        out = ck.matvec_w4a8(xq2, xs2, wo.nibbles, wo.scales, wo.n, wo.k)
    else:  # :743 -> matmul_x -> fused_matvec_w4a16
        if fused and residual is not None:
            return ck.matvec_w4a16_multi(attn, wo.awq_scales, [wo.triple()], wo.k, residuals=[residual])[0]
        out = ck.fused_matvec_w4a16(attn, wo.nibbles, wo.scales, wo.awq_scales, wo.n, wo.k)
    if residual is not None:
        tmp = residual.clone()
        ck.add_inplace(tmp, out)  # :1073
        return tmp
    return out


def gpu_ffn(normed_or_q8, w: GpuLayerWeights, state: GpuInferenceState, use_w4a8: bool,
            residual: Optional[Tensor] = None) -> Tensor:
    """src/gpu_layer.rs:914-996 for SwiGLU with W4 weights at batch 1."""
    fused = state.fused
    wg, wu, wd = w.gate_proj, w.up_proj, w.down_proj
    if use_w4a8:  # :937-947
        if isinstance(normed_or_q8, tuple):
            xq, xs = normed_or_q8
        else:
            xq, xs = ck.quantize_f16_q8(normed_or_q8)
        if fused:
            gate, up = ck.matvec_w4a8_multi(xq, xs, [wg.triple(), wu.triple()], wg.k)
            xq2, xs2, _ = ck.silu_mul_quantize_q8(gate, up)
            if residual is not None:
                return ck.matvec_w4a8_multi(xq2, xs2, [wd.triple()], wd.k, residuals=[residual])[0]
            return ck.matvec_w4a8(xq2, xs2, wd.nibbles, wd.scales, wd.n, wd.k)
        gate = ck.matvec_w4a8(xq, xs, wg.nibbles, wg.scales, wg.n, wg.k)
        up = ck.matvec_w4a8(xq, xs, wu.nibbles, wu.scales, wu.n, wu.k)
        ck.silu_mul_inplace(gate, up)
        xq2, xs2 = ck.quantize_f16_q8(gate)
        out = ck.matvec_w4a8(xq2, xs2, wd.nibbles, wd.scales, wd.n, wd.k)
    else:  # :977-981
        x = normed_or_q8
        same_awq = (wg.awq_scales is None and wu.awq_scales is None)
        if fused and same_awq:
            gate, up = ck.matvec_w4a16_multi(x, None, [wg.triple(), wu.triple()], wg.k)
        else:
            gate = ck.fused_matvec_w4a16(x, wg.nibbles, wg.scales, wg.awq_scales, wg.n, wg.k)
            up = ck.fused_matvec_w4a16(x, wu.nibbles, wu.scales, wu.awq_scales, wu.n, wu.k)
        ck.silu_mul_inplace(gate, up)
        if fused and residual is not None:
            return ck.matvec_w4a16_multi(gate, wd.awq_scales, [wd.triple()], wd.k, residuals=[residual])[0]
        out = ck.fused_matvec_w4a16(gate, wd.nibbles, wd.scales, wd.awq_scales, wd.n, wd.k)
    if residual is not None:
        tmp = residual.clone()
        ck.add_inplace(tmp, out)  # :1082
        return tmp
    return out


def _fused_attention_supported(state: "GpuInferenceState") -> bool:
    return state.head_dim in (64, 128)


def _layer_forward_fused(hidden: Tensor, w: GpuLayerWeights, state: GpuInferenceState, layer_idx: int, d_pos: int,
                         d_seqlen: int, use_w4a8: bool, out: Optional[Tensor] = None, scratch=None,
                         allreduce: bool = False) -> Tensor:
    """Six launches per layer: [RMSNorm + q/k/v GEMV], [RoPE + KV write + attention (+ quantise)], [o_proj GEMV +
    residual], [RMSNorm + gate/up GEMV], [SiLU*up (+ quantise)], [down GEMV + residual].  `scratch` supplies
    pre-allocated buffers (graph capture); `out` receives the new hidden state (may alias `hidden`).  With
    `allreduce` the weights are this rank's tensor-parallel shards and the two row-parallel GEMVs sum their output
    over the ranks inside the kernel."""
    nh, nkv, hd = state.num_heads, state.num_kv_heads, state.head_dim
    dev, f16 = hidden.device, torch.float16
    hidden_size = hidden.numel()
    ffn = w.gate_proj.n
    s = scratch

    def buf(name, shape, dtype=f16, zero=False):
        if s is not None:
            return getattr(s, name)
        return (torch.zeros if zero else torch.empty)(shape, dtype=dtype, device=dev)

    q, k, v = buf("q", (nh, hd)), buf("k", (nkv, hd)), buf("v", (nkv, hd))
    attn = buf("attn", (1, nh * hd))
    gate, up = buf("gate", (1, ffn)), buf("up", (1, ffn))
    h1 = out if out is not None else torch.empty_like(hidden)
    qkv_w = [w.q_proj.triple(), w.k_proj.triple(), w.v_proj.triple()]
    qkv_o = [q.view(1, -1), k.view(1, -1), v.view(1, -1)]
    kc, vc = state.kv_cache.k[layer_idx], state.kv_cache.v[layer_idx]
    max_seq = state.kv_cache.max_seq
    eps, scale = state.norm_eps, float(hd) ** -0.5
    if use_w4a8:
        xq_a, xs_a = buf("xq_a", (nh * hd,), torch.int8), buf("xs_a", (nh * hd // 32,), torch.float32)
        xq_f, xs_f = buf("xq_f", (ffn,), torch.int8), buf("xs_f", (ffn // 32,), torch.float32)
        ck.rmsnorm_matvec_w4a8_multi(hidden, w.input_norm, eps, qkv_w, w.q_proj.k, outs=qkv_o)
        ck.attn_decode_fused(q, k, v, kc, vc, state.rope_cos, state.rope_sin, d_pos, d_seqlen, attn.view(nh, hd), nh, nkv,
                             hd, max_seq, scale, out_q=xq_a, out_scales=xs_a)
        gemv8 = ck.matvec_w4a8_allreduce if allreduce else ck.matvec_w4a8_multi
        gemv8(xq_a, xs_a, [w.o_proj.triple()], w.o_proj.k, outs=[h1], residuals=[hidden])
        if state.fuse_silu and state.convert_in_down_prologue:
            ck.rmsnorm_gateup_silu(h1, w.post_attn_norm, eps, None, w.gate_proj.triple(), w.up_proj.triple(), w.gate_proj.k,
                                   True, mid=gate)
            ck.quantize_matvec_w4a8_multi(gate, None, [w.down_proj.triple()], w.down_proj.k, outs=[h1], residuals=[h1],
                                          allreduce=allreduce)
            return h1
        if state.fuse_silu:
            # SiLU*up in the gate/up epilogue; the CTA that completes a 32-wide group of it writes the group's int8 codes
            cnt = buf("pq_cnt", (ffn // 32,), torch.int32, zero=True)
            ck.rmsnorm_gateup_silu(h1, w.post_attn_norm, eps, None, w.gate_proj.triple(), w.up_proj.triple(), w.gate_proj.k,
                                   True, mid=gate, quant={"xq": xq_f, "xs": xs_f, "counters": cnt})
            gemv8(xq_f, xs_f, [w.down_proj.triple()], w.down_proj.k, outs=[h1], residuals=[h1])
            return h1
        ck.rmsnorm_matvec_w4a8_multi(h1, w.post_attn_norm, eps, [w.gate_proj.triple(), w.up_proj.triple()], w.gate_proj.k,
                                     outs=[gate, up])
        ck.silu_mul_quantize_q8(gate, up, xq=xq_f, scales=xs_f)
        gemv8(xq_f, xs_f, [w.down_proj.triple()], w.down_proj.k, outs=[h1], residuals=[h1])
    else:
        ck.rmsnorm_matvec_w4a16_multi(hidden, w.input_norm, eps, w.q_proj.awq_scales, qkv_w, w.q_proj.k, outs=qkv_o)
        ck.attn_decode_fused(q, k, v, kc, vc, state.rope_cos, state.rope_sin, d_pos, d_seqlen, attn.view(nh, hd), nh, nkv,
                             hd, max_seq, scale)
        gemv16 = ck.matvec_w4a16_allreduce if allreduce else ck.matvec_w4a16_multi
        gemv16(attn, w.o_proj.awq_scales, [w.o_proj.triple()], w.o_proj.k, outs=[h1], residuals=[hidden])
        xq_f, xs_f = buf("xq_f", (ffn,), torch.int8), buf("xs_f", (ffn // 32,), torch.float32)
        xlo_f = buf("xlo_f", (ffn,), torch.uint8)
        down16 = ck.matvec_w4a16_planes_allreduce if allreduce else ck.matvec_w4a16_planes_multi
        if state.fuse_silu and state.convert_in_down_prologue:
            ck.rmsnorm_gateup_silu(h1, w.post_attn_norm, eps, w.gate_proj.awq_scales, w.gate_proj.triple(),
                                   w.up_proj.triple(), w.gate_proj.k, False, mid=gate)
            gemv16(gate, w.down_proj.awq_scales, [w.down_proj.triple()], w.down_proj.k, outs=[h1], residuals=[h1])
            return h1
        if state.fuse_silu:
            # ... or the group's 16-bit fixed-point planes, as the stand-alone SiLU kernel below would
            cnt = buf("pq_cnt", (ffn // 32,), torch.int32, zero=True)
            ck.rmsnorm_gateup_silu(h1, w.post_attn_norm, eps, w.gate_proj.awq_scales, w.gate_proj.triple(),
                                   w.up_proj.triple(), w.gate_proj.k, False, mid=gate,
                                   quant={"xlo": xlo_f, "xhi": xq_f, "xs": xs_f, "counters": cnt,
                                          "down_awq": w.down_proj.awq_scales})
            down16(xlo_f, xq_f, xs_f, [w.down_proj.triple()], w.down_proj.k, outs=[h1], residuals=[h1])
            return h1
        ck.rmsnorm_matvec_w4a16_multi(h1, w.post_attn_norm, eps, w.gate_proj.awq_scales,
                                      [w.gate_proj.triple(), w.up_proj.triple()], w.gate_proj.k, outs=[gate, up])
        # the fixed-point form of silu(gate)*up is produced once here instead of by every CTA of the GEMV
        ck.silu_mul_x16(gate, up, w.down_proj.awq_scales, x_lo=xlo_f, x_hi=xq_f, scales=xs_f)
        down16(xlo_f, xq_f, xs_f, [w.down_proj.triple()], w.down_proj.k, outs=[h1], residuals=[h1])
    return h1


def gpu_layer_forward_decode(hidden: Tensor, layer_idx: int, state: GpuInferenceState, pos: int,
                             parallel_attn_ffn: bool = False, layer_importance: float = 0.0,
                             d_pos: Optional[int] = None, d_seqlen: Optional[int] = None) -> Tensor:
    """src/gpu_layer.rs:1005-1084: one token through one layer.  hidden [1, hidden] f16 -> same shape.

    `d_pos` / `d_seqlen` are device addresses of the position and valid-length scalars; when omitted the
    state's own scalars are set from `pos` (eager use)."""
    if parallel_attn_ffn:
        raise NotImplementedError("parallel attention+FFN blocks are outside the quantized Llama decode path")
    use_w4a8 = state.routing.use_w4a8(layer_importance)
    w = state.layer_weights[layer_idx]
    if d_pos is None:
        state.set_position(pos)
        d_pos, d_seqlen = state.d_pos.data_ptr(), state.d_seqlen.data_ptr()
    eps = state.norm_eps
    same_awq = (w.q_proj.awq_scales is w.k_proj.awq_scales is w.v_proj.awq_scales) and \
        (w.gate_proj.awq_scales is w.up_proj.awq_scales)
    if state.fused and _fused_attention_supported(state) and (use_w4a8 or same_awq):
        return _layer_forward_fused(hidden, w, state, layer_idx, d_pos, d_seqlen, use_w4a8)
    if state.fused and use_w4a8:
        xq, xs, _ = ck.rmsnorm_quantize_q8(hidden, w.input_norm, eps)
        h = gpu_attn_decode((xq, xs), w, state, layer_idx, d_pos, d_seqlen, True, residual=hidden)
        xq, xs, _ = ck.rmsnorm_quantize_q8(h, w.post_attn_norm, eps)
        return gpu_ffn((xq, xs), w, state, True, residual=h)
    normed = ck.fused_rms_norm(hidden, w.input_norm, eps)  # :1032-1038
    h = gpu_attn_decode(normed, w, state, layer_idx, d_pos, d_seqlen, use_w4a8, residual=hidden)
    normed2 = ck.fused_rms_norm(h, w.post_attn_norm, eps)  # :1074-1080
    return gpu_ffn(normed2, w, state, use_w4a8, residual=h)



def gpu_layer_forward_prefill(hidden: Tensor, layer_idx: int, state: GpuInferenceState, start_pos: int) -> Tensor:
    """src/gpu_layer.rs:1086-1160 with gpu_attn_prefill (:777-890) and the batch > 1 branch of gpu_ffn (:977-996) for
    W4 weights: all S prompt positions of one sequence through one layer.  hidden [S, hidden] f16 -> same shape; the
    K/V cache of the layer receives positions start_pos .. start_pos + S - 1.

    The reference dequantises every projection to f16 and calls a dense GEMM, runs RMSNorm once per token and an
    unfused masked attention; here the projections are the tensor-core GEMM on the packed weights (q/k/v and gate/up one
    launch each per 64-row slice), RMSNorm / KV write / causal attention are one launch each.  Like the reference's
    prefill, every layer runs on 16-bit activations (the int8 route is a batch-1 path, :1017-1025)."""
    if hidden.dim() != 2:
        raise ValueError("hidden must be [S, hidden]")
    w = state.layer_weights[layer_idx]
    nh, nkv, hd = state.num_heads, state.num_kv_heads, state.head_dim
    S = hidden.shape[0]
    max_seq = state.kv_cache.max_seq
    if start_pos < 0 or start_pos + S > max_seq:
        raise ValueError("the block does not fit the K/V cache")
    eps, scale = state.norm_eps, float(hd) ** -0.5
    normed = ck.rms_norm_rows(hidden, w.input_norm, eps)
    q, k, v = matmul_x_multi(normed, [w.q_proj, w.k_proj, w.v_proj])
    ck.fused_rope_prefill(q, k, state.rope_cos, state.rope_sin, S, nh, nkv, hd, start_pos)
    kc, vc = state.kv_cache.k[layer_idx], state.kv_cache.v[layer_idx]
    ck.kv_cache_write_rows(k.view(S, nkv, hd), kc, v.view(S, nkv, hd), vc, start_pos, nkv, hd, max_seq)
    attn = ck.attn_prefill_causal(q, kc, vc, start_pos, nh, nkv, hd, max_seq, scale)
    h1 = matmul_x(attn, w.o_proj)
    normed2 = ck.add_rms_norm_rows(h1, hidden, w.post_attn_norm, eps)  # residual add + norm in one launch
    gate, up = matmul_x_multi(normed2, [w.gate_proj, w.up_proj])
    ck.silu_mul_inplace(gate, up)
    out = matmul_x(gate, w.down_proj)
    ck.add_inplace_any(out, h1)
    return out


@dataclass
class BatchedKvCache:
    """Static K/V caches of B independent sequences: per layer k / v [B, nkv, max_seq, hd] f16 (the reference has no
    batched decode; this is the single-sequence layout of src/decode_graph.rs:183-184 with a batch dimension in front)."""

    k: List[Tensor]
    v: List[Tensor]
    batch: int
    max_seq: int

    @staticmethod
    def zeros(num_layers: int, batch: int, num_kv_heads: int, max_seq: int, head_dim: int, device="cuda") -> "BatchedKvCache":
        mk = lambda: [torch.zeros((batch, num_kv_heads, max_seq, head_dim), dtype=torch.float16, device=device)
                      for _ in range(num_layers)]
        return BatchedKvCache(mk(), mk(), batch, max_seq)


@dataclass
class BatchedDecodeScratch:
    """Every intermediate of gpu_layer_forward_decode_batch for a fixed batch, so that a step allocates nothing (and can
    be recorded into a CUDA graph)."""

    normed: Tensor
    q: Tensor
    k: Tensor
    v: Tensor
    attn: Tensor
    h1: Tensor
    gate: Tensor
    up: Tensor
    out: List[Tensor]   # two output rows buffers, alternated between layers (a layer reads the previous layer's output)
    gemm: Tensor        # workspace of the batched GEMM (largest of the four projection groups)

    @staticmethod
    def make(state: GpuInferenceState, batch: int, hidden: int, ffn: int, device="cuda") -> "BatchedDecodeScratch":
        nh, nkv, hd = state.num_heads, state.num_kv_heads, state.head_dim
        f16 = torch.float16
        z = lambda n: torch.zeros((batch, n), dtype=f16, device=device)
        groups = [([nh * hd, nkv * hd, nkv * hd], hidden), ([hidden], nh * hd), ([ffn, ffn], hidden), ([hidden], ffn)]
        nbytes = max(ck.gemm_w4a16_multi_scratch_bytes(min(batch, 64), ns, k) for ns, k in groups) if batch > 1 else 0
        return BatchedDecodeScratch(z(hidden), z(nh * hd), z(nkv * hd), z(nkv * hd), z(nh * hd), z(hidden), z(ffn), z(ffn),
                                    [z(hidden), z(hidden)], torch.empty(max(16, nbytes), dtype=torch.uint8, device=device))


def gpu_layer_forward_decode_batch(hidden: Tensor, layer_idx: int, state: GpuInferenceState, kv: BatchedKvCache,
                                   d_pos: Tensor, d_seqlen: Tensor, scratch: Optional[BatchedDecodeScratch] = None,
                                   residual: Optional[Tensor] = None, defer_add: bool = False):
    """One decode step of B independent sequences through one layer: hidden [B, hidden] f16 -> same shape.  Row b is the
    next token of sequence b at position d_pos[b] (int32 device tensors [B]); kv holds the sequences' caches.

    The projections are the tensor-core GEMM on the packed weights (B <= 64 rows per launch; q/k/v and gate/up one launch
    each), RoPE + K/V write + attention of all sequences is one launch of the fused decode kernel, RMSNorm one launch
    over the rows.  16-bit activations on every layer, as in prefill.  Row b equals the single-sequence decode of that
    sequence within the tolerance that separates the tensor-core GEMM from the integer GEMV.  With `scratch` nothing is
    allocated and the result is one of scratch.out (alternating with the layer index).

    The residual adds ride on the RMSNorm launches (add_rms_norm_rows, same bits as the separate kernels).  For the
    add at the end of a layer that needs the next layer's norm: with defer_add the layer returns (out, h1) without
    adding, and the next layer is called with hidden = out, residual = h1 and adds them (in place, into `hidden`)
    inside its first launch."""
    if hidden.dim() != 2 or hidden.shape[0] != kv.batch:
        raise ValueError("hidden must be [batch, hidden] with the cache's batch")
    w = state.layer_weights[layer_idx]
    nh, nkv, hd = state.num_heads, state.num_kv_heads, state.head_dim
    eps, scale = state.norm_eps, float(hd) ** -0.5
    s = scratch
    ws = None if s is None else s.gemm
    if residual is not None:
        normed = ck.add_rms_norm_rows(hidden, residual, w.input_norm, eps, out=None if s is None else s.normed)
    else:
        normed = ck.rms_norm_rows(hidden, w.input_norm, eps, out=None if s is None else s.normed)
    q, k, v = matmul_x_multi(normed, [w.q_proj, w.k_proj, w.v_proj], ws, None if s is None else [s.q, s.k, s.v])
    attn = ck.attn_decode_fused_batch(q, k, v, kv.k[layer_idx], kv.v[layer_idx], state.rope_cos, state.rope_sin, d_pos,
                                      d_seqlen, nh, nkv, hd, kv.max_seq, scale, out=None if s is None else s.attn)
    h1 = matmul_x(attn, w.o_proj, ws, None if s is None else s.h1)
    normed2 = ck.add_rms_norm_rows(h1, hidden, w.post_attn_norm, eps, out=None if s is None else s.normed)
    gate, up = matmul_x_multi(normed2, [w.gate_proj, w.up_proj], ws, None if s is None else [s.gate, s.up])
    ck.silu_mul_inplace(gate, up)
    out = matmul_x(gate, w.down_proj, ws, None if s is None else s.out[layer_idx & 1])
    if defer_add:
        return out, h1
    ck.add_inplace_any(out, h1)
    return out
