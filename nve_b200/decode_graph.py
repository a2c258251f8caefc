"""Static decode graph: pre-allocated buffers, one CUDA-graph capture of the whole layer stack, replay.

Mirrors the reference's src/decode_graph.rs: `StaticDecodeGraph::capture` (:138-370) records, for every
layer, the kernel sequence into the library's process-global graph (nve_graph_*), and `replay` (:382-404)
copies the input row into `hidden_buf`, sets pos / seq_len and launches.  Two differences, both on the
caller side of the C ABI:
  * the reference records W4A16 kernels only (:218-342); here each layer is recorded on the route its
    importance score selects (src/gpu_layer.rs:1017-1025), so a mixed W4A8 / W4A16 stack replays as one graph;
  * the fused entry points shorten a layer from 12 recorded steps to 6 launches.
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

    q: Tensor
    k: Tensor
    v: Tensor
    attn: Tensor
    gate: Tensor
    up: Tensor
    xq_a: Tensor
    xs_a: Tensor
    xq_f: Tensor
    xs_f: Tensor
    xlo_f: Tensor
    pq_cnt: Tensor  # per 32-wide group of the FFN activation: values written so far (five-launch layer)


class StaticDecodeGraph:
    """One captured decode step over all layers of a GpuInferenceState."""

    def __init__(self, state: GpuInferenceState, hidden_size: int, ffn_size: int, importance: Sequence[float],
                 allreduce: bool = False, lm_head=None):
        """`lm_head` = (weights, final_norm, kind) appends the final RMSNorm and the lm_head GEMV that the reference
        runs on the host (src/paged_model.rs:1424-1433): kind "w4a16" / "w4a8" with a GpuW4 (logits f32, one fused
        launch) or "f16" with a dense [vocab, hidden] f16 tensor (RMSNorm launch + nve_matvec_f16, logits f16)."""
        self.state = state
        self.lm_head = lm_head
        self.logits = None
        self.allreduce = allreduce  # tensor parallel: `state` holds this rank's shards (ffn_size is the local FFN width)
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
            q=torch.zeros((nh, hd), dtype=f16, device=dev),
            k=torch.zeros((nkv, hd), dtype=f16, device=dev),
            v=torch.zeros((nkv, hd), dtype=f16, device=dev),
            attn=torch.zeros((1, nh * hd), dtype=f16, device=dev),
            gate=torch.zeros((1, ffn_size), dtype=f16, device=dev),
            up=torch.zeros((1, ffn_size), dtype=f16, device=dev),
            xq_a=torch.zeros(nh * hd, dtype=torch.int8, device=dev),
            xs_a=torch.zeros(nh * hd // 32, dtype=torch.float32, device=dev),
            xq_f=torch.zeros(ffn_size, dtype=torch.int8, device=dev),
            xs_f=torch.zeros(ffn_size // 32, dtype=torch.float32, device=dev),
            xlo_f=torch.zeros(ffn_size, dtype=torch.uint8, device=dev),
            pq_cnt=torch.zeros(max(1, ffn_size // 32), dtype=torch.int32, device=dev),
        )
        self.s = s
        self.routes: List[bool] = [state.routing.use_w4a8(x) for x in self.importance]
        self.launches_per_replay = 0
        self.captured = False
        if lm_head is not None:
            w, _norm, kind = lm_head
            if kind == "f16":
                self.logits = torch.zeros((1, w.shape[0]), dtype=f16, device=dev)
                self._normed = torch.zeros((1, hidden_size), dtype=f16, device=dev)
            else:
                self.logits = torch.zeros((1, w.n), dtype=torch.float32, device=dev)

    # ------------------------------------------------------------------ recording
    def _record_lm_head(self) -> None:
        w, norm, kind = self.lm_head
        eps = self.state.norm_eps
        if kind == "f16":
            ck.fused_rms_norm_into(self.hidden_buf, norm, self._normed, eps)
            ck.fused_matvec_into(self._normed, w, self.logits, w.shape[0], w.shape[1])
        elif kind == "w4a8":
            ck.rmsnorm_matvec_w4a8_multi(self.hidden_buf, norm, eps, [w.triple()], w.k, out_dtype=torch.float32,
                                         outs=[self.logits])
        else:
            ck.rmsnorm_matvec_w4a16_multi(self.hidden_buf, norm, eps, w.awq_scales, [w.triple()], w.k,
                                          out_dtype=torch.float32, outs=[self.logits])

    def _record_layer(self, li: int, d_pos: int, d_seqlen: int) -> None:
        from .gpu_layer import _layer_forward_fused

        st = self.state
        _layer_forward_fused(self.hidden_buf, st.layer_weights[li], st, li, d_pos, d_seqlen, self.routes[li],
                             out=self.hidden_buf, scratch=self.s, allreduce=self.allreduce)

    def capture(self) -> None:
        """src/decode_graph.rs:138-370."""
        ck.graph_init()
        before = ck.launch_count()
        ck.graph_begin_capture()
        try:
            d_pos, d_seqlen = ck.graph_d_pos_ptr(), ck.graph_d_seqlen_ptr()
            for li in range(len(self.state.layer_weights)):
                self._record_layer(li, d_pos, d_seqlen)
            if self.lm_head is not None:
                self._record_lm_head()
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


class PersistentDecode:
    """The same decode step as `StaticDecodeGraph`, run by ONE persistent kernel (nve_b200_decode_step) instead of
    five or six launches per layer.  The launch is recorded into the library's graph like the layer sequence is, so
    `replay` / `replay_resident` drive it through the same pinned position scalars; the hidden state it leaves is
    bit-identical to the graph of separate launches.  `lm_head` = (GpuW4, final_norm weight, use_w4a8) adds the device-side
    final RMSNorm + lm_head GEMV; logits land in `self.logits` (f32)."""

    def __init__(self, state: GpuInferenceState, hidden_size: int, ffn_size: int, importance: Sequence[float],
                 lm_head=None):
        import ctypes as C

        from . import _ffi

        self.state = state
        self.hidden_size, self.ffn_size = hidden_size, ffn_size
        self.importance = list(importance)
        self.routes: List[bool] = [state.routing.use_w4a8(x) for x in self.importance]
        dev = state.rope_cos.device
        self.hidden_buf = torch.zeros((1, hidden_size), dtype=torch.float16, device=dev)
        m = _ffi.DecodeModel()
        m.hidden, m.ffn = hidden_size, ffn_size
        m.num_heads, m.num_kv_heads, m.head_dim = state.num_heads, state.num_kv_heads, state.head_dim
        m.max_seq, m.num_layers = state.kv_cache.max_seq, len(state.layer_weights)
        m.norm_eps, m.attn_scale = state.norm_eps, float(state.head_dim) ** -0.5
        m.rope_cos, m.rope_sin = state.rope_cos.data_ptr(), state.rope_sin.data_ptr()
        self.logits = None
        self._keep = []
        if lm_head is not None:
            w, final_norm, use_w4a8 = lm_head
            self.logits = torch.zeros(w.n, dtype=torch.float32, device=dev)
            m.final_norm, m.lm_nibbles, m.lm_scales = final_norm.data_ptr(), w.nibbles.data_ptr(), w.scales.data_ptr()
            m.logits, m.vocab, m.lm_use_w4a8 = self.logits.data_ptr(), w.n, int(bool(use_w4a8))
            self._keep += [w, final_norm]
        self.model = m
        descs = (_ffi.DecodeLayer * m.num_layers)()
        for li, lw in enumerate(state.layer_weights):
            d = descs[li]
            projs = [lw.q_proj, lw.k_proj, lw.v_proj, lw.o_proj, lw.gate_proj, lw.up_proj, lw.down_proj]
            for j, w in enumerate(projs):
                d.nibbles[j], d.scales[j] = w.nibbles.data_ptr(), w.scales.data_ptr()
            if not (lw.q_proj.awq_scales is lw.k_proj.awq_scales is lw.v_proj.awq_scales) or \
                    lw.gate_proj.awq_scales is not lw.up_proj.awq_scales:
                raise ValueError("q/k/v (and gate/up) must share one activation multiplier")
            for j, w in enumerate((lw.q_proj, lw.o_proj, lw.gate_proj, lw.down_proj)):
                d.awq[j] = w.awq_scales.data_ptr() if w.awq_scales is not None else None
            d.input_norm, d.post_attn_norm = lw.input_norm.data_ptr(), lw.post_attn_norm.data_ptr()
            d.k_cache, d.v_cache = state.kv_cache.k[li].data_ptr(), state.kv_cache.v[li].data_ptr()
            d.use_w4a8 = int(self.routes[li])
        raw = torch.frombuffer(bytearray(bytes(descs)), dtype=torch.uint8)
        self.layers_dev = raw.to(dev)
        nbytes = ck.decode_step_workspace_bytes(m)
        self.workspace = torch.zeros(nbytes + 256, dtype=torch.uint8, device=dev)
        off = (-self.workspace.data_ptr()) % 256
        self.workspace = self.workspace[off:off + nbytes]
        ck.decode_step_init(self.workspace)
        self.launches_per_replay = 1
        self.captured = False

    def step(self, d_pos: int, d_seqlen: int) -> None:
        """Enqueue the kernel on the current (or capture) stream with device position scalars."""
        ck.decode_step(self.model, self.layers_dev, self.hidden_buf, d_pos, d_seqlen, self.workspace)

    def capture(self) -> None:
        ck.graph_init()
        ck.graph_begin_capture()
        try:
            self.step(ck.graph_d_pos_ptr(), ck.graph_d_seqlen_ptr())
        finally:
            ck.graph_end_capture()
        if not ck.graph_ready():
            raise RuntimeError("decode graph instantiation failed")
        self.captured = True

    def replay(self, hidden_in: Tensor, pos: int, copy_out: bool = True) -> Optional[Tensor]:
        if not self.captured:
            raise RuntimeError("capture() first")
        ck.device_copy(self.hidden_buf, hidden_in)
        ck.graph_launch(pos, min(pos + 1, self.state.kv_cache.max_seq))
        return self.hidden_buf.clone() if copy_out else None

    def replay_resident(self, pos: int) -> None:
        ck.graph_launch(pos, min(pos + 1, self.state.kv_cache.max_seq))

    def error(self, reset: bool = False) -> int:
        return ck.decode_step_error(self.workspace, reset)

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
