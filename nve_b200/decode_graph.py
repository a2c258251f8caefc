"""Static decode graph: pre-allocated buffers, one CUDA-graph capture of the whole layer stack, replay.

Mirrors the reference's src/decode_graph.rs: `StaticDecodeGraph::capture` (:138-370) records, for every
layer, the kernel sequence into the library's process-global graph (nve_graph_*), and `replay` (:382-404)
copies the input row into `hidden_buf`, sets pos / seq_len and launches.  Two differences, both on the
caller side of the C ABI:
  * the reference records W4A16 kernels only (:218-342); here each layer is recorded on the route its
    importance score selects (src/gpu_layer.rs:1017-1025), so a mixed W4A8 / W4A16 stack replays as one graph;
  * the fused entry points shorten a layer from 12 recorded steps to 10 launches.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from . import cuda_kernels as ck
from .gpu_layer import GpuInferenceState

Tensor = torch.Tensor


@dataclass
class _LayerScratch:
    """Per-layer scratch of src/decode_graph.rs:60-71, plus the int8 staging of the W4A8 route."""

    normed: Tensor
    q: Tensor
    k: Tensor
    v: Tensor
    attn: Tensor
    gate: Tensor
    up: Tensor
    xq_h: Tensor
    xs_h: Tensor
    xq_a: Tensor
    xs_a: Tensor
    xq_f: Tensor
    xs_f: Tensor


class StaticDecodeGraph:
    """One captured decode step over all layers of a GpuInferenceState."""

    def __init__(self, state: GpuInferenceState, hidden_size: int, ffn_size: int, importance: Sequence[float]):
        self.state = state
        self.hidden_size = hidden_size
        self.ffn_size = ffn_size
        self.importance = list(importance)
        dev = state.rope_cos.device
        f16 = torch.float16
        nh, nkv, hd = state.num_heads, state.num_kv_heads, state.head_dim
        self.hidden_buf = torch.zeros((1, hidden_size), dtype=f16, device=dev)
        self.scratch: List[_LayerScratch] = []
        # one scratch set is enough: layers run back to back on one stream
        s = _LayerScratch(
            normed=torch.zeros((1, hidden_size), dtype=f16, device=dev),
            q=torch.zeros((nh, hd), dtype=f16, device=dev),
            k=torch.zeros((nkv, hd), dtype=f16, device=dev),
            v=torch.zeros((nkv, hd), dtype=f16, device=dev),
            attn=torch.zeros((1, nh * hd), dtype=f16, device=dev),
            gate=torch.zeros((1, ffn_size), dtype=f16, device=dev),
            up=torch.zeros((1, ffn_size), dtype=f16, device=dev),
            xq_h=torch.zeros(hidden_size, dtype=torch.int8, device=dev),
            xs_h=torch.zeros(hidden_size // 32, dtype=torch.float32, device=dev),
            xq_a=torch.zeros(nh * hd, dtype=torch.int8, device=dev),
            xs_a=torch.zeros(nh * hd // 32, dtype=torch.float32, device=dev),
            xq_f=torch.zeros(ffn_size, dtype=torch.int8, device=dev),
            xs_f=torch.zeros(ffn_size // 32, dtype=torch.float32, device=dev),
        )
        self.s = s
        self.routes: List[bool] = [state.routing.use_w4a8(x) for x in self.importance]
        self.launches_per_replay = 0
        self.captured = False

    # ------------------------------------------------------------------ recording
    def _record_layer(self, li: int, d_pos: int, d_seqlen: int) -> None:
        st, s = self.state, self.s
        w = st.layer_weights[li]
        nh, nkv, hd = st.num_heads, st.num_kv_heads, st.head_dim
        h = self.hidden_buf
        kc, vc = st.kv_cache.k[li], st.kv_cache.v[li]
        max_seq = st.kv_cache.max_seq
        eps = st.norm_eps
        qv, kv, vv = s.q.view(1, -1), s.k.view(1, -1), s.v.view(1, -1)
        if self.routes[li]:
            ck.rmsnorm_quantize_q8(h, w.input_norm, eps, xq=s.xq_h, scales=s.xs_h)
            ck.matvec_w4a8_multi(s.xq_h, s.xs_h, [w.q_proj.triple(), w.k_proj.triple(), w.v_proj.triple()], w.q_proj.k,
                                 outs=[qv, kv, vv])
        else:
            ck.fused_rms_norm_into(h, w.input_norm, s.normed, eps)
            ck.matvec_w4a16_multi(s.normed, w.q_proj.awq_scales,
                                  [w.q_proj.triple(), w.k_proj.triple(), w.v_proj.triple()], w.q_proj.k, outs=[qv, kv, vv])
        ck.rope_decode_dyn_inplace(s.q, s.k, st.rope_cos, st.rope_sin, nh, nkv, hd, d_pos)
        ck.kv_cache_write(s.k, kc, s.v, vc, d_pos, nkv, hd, max_seq)
        ck.flash_decode_dyn_into(s.q, kc, vc, s.attn.view(nh, hd), nh, nkv, d_seqlen, hd, float(hd) ** -0.5, max_seq)
        if self.routes[li]:
            xq, xs = s.xq_a, s.xs_a
            ck._ffi.check("nve_b200_quantize_q8", ck._lib().nve_b200_quantize_q8(
                s.attn.data_ptr(), xq.data_ptr(), xs.data_ptr(), s.attn.numel(), ck.NVE_DT_F16, ck.stream()))
            ck.matvec_w4a8_multi(xq, xs, [w.o_proj.triple()], w.o_proj.k, outs=[h], residuals=[h])
            ck.rmsnorm_quantize_q8(h, w.post_attn_norm, eps, xq=s.xq_h, scales=s.xs_h)
            ck.matvec_w4a8_multi(s.xq_h, s.xs_h, [w.gate_proj.triple(), w.up_proj.triple()], w.gate_proj.k,
                                 outs=[s.gate, s.up])
            ck.silu_mul_quantize_q8(s.gate, s.up, xq=s.xq_f, scales=s.xs_f)
            ck.matvec_w4a8_multi(s.xq_f, s.xs_f, [w.down_proj.triple()], w.down_proj.k, outs=[h], residuals=[h])
        else:
            ck.matvec_w4a16_multi(s.attn, w.o_proj.awq_scales, [w.o_proj.triple()], w.o_proj.k, outs=[h], residuals=[h])
            ck.fused_rms_norm_into(h, w.post_attn_norm, s.normed, eps)
            ck.matvec_w4a16_multi(s.normed, w.gate_proj.awq_scales, [w.gate_proj.triple(), w.up_proj.triple()],
                                  w.gate_proj.k, outs=[s.gate, s.up])
            ck.silu_mul_inplace(s.gate, s.up)
            ck.matvec_w4a16_multi(s.gate, w.down_proj.awq_scales, [w.down_proj.triple()], w.down_proj.k, outs=[h],
                                  residuals=[h])

    def capture(self) -> None:
        """src/decode_graph.rs:138-370."""
        ck.graph_init()
        before = ck.launch_count()
        ck.graph_begin_capture()
        try:
            d_pos, d_seqlen = ck.graph_d_pos_ptr(), ck.graph_d_seqlen_ptr()
            for li in range(len(self.state.layer_weights)):
                self._record_layer(li, d_pos, d_seqlen)
        finally:
            ck.graph_end_capture()
        self.launches_per_replay = ck.launch_count() - before
        if not ck.graph_ready():
            raise RuntimeError("decode graph instantiation failed")
        self.captured = True

    def replay(self, hidden_in: Tensor, pos: int, copy_out: bool = True) -> Optional[Tensor]:
        """src/decode_graph.rs:382-404: copy the input row in, launch with (pos, min(pos+1, max_seq))."""
        if not self.captured:
            raise RuntimeError("capture() first")
        ck.device_copy(self.hidden_buf, hidden_in)
        ck.graph_launch(pos, min(pos + 1, self.state.kv_cache.max_seq))
        return self.hidden_buf.clone() if copy_out else None

    def replay_resident(self, pos: int) -> None:
        """Launch on the current contents of `hidden_buf` (no input copy, no output clone)."""
        ck.graph_launch(pos, min(pos + 1, self.state.kv_cache.max_seq))

    def destroy(self) -> None:
        ck.graph_destroy()
        self.captured = False


class CapturedSequence:
    """Record an arbitrary sequence of library launches into the library's (single, process-global) graph and
    replay it.  Used by the measurement harness to time subsets of the decode step (e.g. the GEMV launches
    alone) with exactly the launch parameters the full step uses."""

    def __init__(self, record_fn):
        ck.graph_init()
        before = ck.launch_count()
        ck.graph_begin_capture()
        try:
            record_fn(ck.graph_d_pos_ptr(), ck.graph_d_seqlen_ptr())
        finally:
            ck.graph_end_capture()
        self.launches = ck.launch_count() - before
        if not ck.graph_ready():
            raise RuntimeError("graph instantiation failed")

    def replay(self, pos: int, seq_len: int) -> None:
        ck.graph_launch(pos, seq_len)

    def destroy(self) -> None:
        ck.graph_destroy()
