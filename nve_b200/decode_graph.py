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
    xlo_f: Tensor


class StaticDecodeGraph:
    """One captured decode step over all layers of a GpuInferenceState."""

    def __init__(self, state: GpuInferenceState, hidden_size: int, ffn_size: int, importance: Sequence[float],
                 allreduce: bool = False):
        self.state = state
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
            xlo_f=torch.zeros(ffn_size, dtype=torch.uint8, device=dev),
        )
        self.s = s
        self.routes: List[bool] = [state.routing.use_w4a8(x) for x in self.importance]
        self.launches_per_replay = 0
        self.captured = False

    # ------------------------------------------------------------------ recording
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
