"""Host-side mirror of the reference's src/cuda_kernels.rs wrappers, over torch CUDA tensors.

Each function keeps the name, argument order and meaning of the Rust wrapper it mirrors (cited per
function) so that call sites read like src/gpu_layer.rs / src/decode_graph.rs.  torch is used only for
device memory and streams; every computation is a call through the C ABI of libnve_kernels.so with raw
device pointers.  There is no fallback: without the library these functions raise.

Differences from the Rust wrappers, all on the host side:
  * errors recorded by the library are raised as NveKernelError instead of being ignored;
  * outputs are allocated with torch.empty (the Rust side uses Tensor::zeros, an extra fill kernel);
  * additive wrappers (bf16 I/O, fused prologues, multi-matrix GEMVs) sit at the end of the file.
"""
from __future__ import annotations

import contextlib
import ctypes as C
import threading
from typing import Optional, Sequence, Tuple

import torch

from . import _ffi
from ._ffi import NVE_DT_BF16, NVE_DT_F16, NVE_DT_F32, W4Matrix

Tensor = torch.Tensor
_tls = threading.local()


# --------------------------------------------------------------------------- stream handling
def stream() -> int:
    """src/cuda_kernels.rs:41-44: the capture stream while a graph is being recorded, else the stream
    the caller is working on (torch's current stream; the Rust side uses the legacy default stream)."""
    s = getattr(_tls, "capture_stream", None)
    if s is not None:
        return s
    return torch.cuda.current_stream().cuda_stream


def set_graph_capture_stream(s: int) -> None:
    """src/cuda_kernels.rs:46-49."""
    _tls.capture_stream = int(s) if s else None


def clear_graph_capture_stream() -> None:
    """src/cuda_kernels.rs:51-53."""
    _tls.capture_stream = None


# --------------------------------------------------------------------------- pointer helpers
_TORCH_DT = {torch.float16: NVE_DT_F16, torch.bfloat16: NVE_DT_BF16, torch.float32: NVE_DT_F32}


def _ptr(t: Optional[Tensor], dtype=None, name: str = "tensor") -> Optional[int]:
    """Device address of a contiguous CUDA tensor (src/cuda_kernels.rs:300-339 does the same for candle)."""
    if t is None:
        return None
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    if dtype is not None:
        ok = t.dtype in dtype if isinstance(dtype, (tuple, list)) else t.dtype == dtype
        if not ok:
            raise TypeError(f"{name} has dtype {t.dtype}, expected {dtype}")
    return t.data_ptr()


def _dt(t: Tensor) -> int:
    try:
        return _TORCH_DT[t.dtype]
    except KeyError:
        raise TypeError(f"unsupported dtype {t.dtype}") from None


def _lib():
    return _ffi.load()


_Q8 = (torch.int8, torch.uint8)
_F16 = torch.float16


# --------------------------------------------------------------------------- reference wrappers
def fused_rms_norm(x: Tensor, weight: Tensor, eps: float) -> Tensor:
    """src/cuda_kernels.rs:351-367."""
    out = torch.empty_like(x)
    fused_rms_norm_into(x, weight, out, eps)
    return out


def fused_rms_norm_into(x: Tensor, weight: Tensor, out: Tensor, eps: float) -> None:
    """src/cuda_kernels.rs:707-715."""
    _lib().nve_rms_norm_f16(_ptr(x, _F16, "x"), _ptr(weight, _F16, "weight"), _ptr(out, _F16, "out"), x.numel(),
                            float(eps), stream())
    _ffi.check_last("nve_rms_norm_f16")


def fused_layer_norm(x: Tensor, weight: Tensor, bias: Optional[Tensor], eps: float) -> Tensor:
    """src/cuda_kernels.rs:373-399."""
    out = torch.empty_like(x)
    _lib().nve_layer_norm_f16(_ptr(x, _F16), _ptr(weight, _F16), _ptr(bias, _F16), _ptr(out), x.numel(), float(eps),
                              stream())
    _ffi.check_last("nve_layer_norm_f16")
    return out


def fused_rope_decode(q: Tensor, k: Tensor, cos_row: Tensor, sin_row: Tensor, num_heads: int, num_kv_heads: int,
                      head_dim: int) -> None:
    """src/cuda_kernels.rs:405-431: rotates q [nh,hd] and k [nkv,hd] in place."""
    _lib().nve_rope_f16_decode(_ptr(q, _F16, "q"), _ptr(k, _F16, "k"), _ptr(cos_row, _F16), _ptr(sin_row, _F16),
                               num_heads, num_kv_heads, head_dim, stream())
    _ffi.check_last("nve_rope_f16_decode")


def fused_rope_prefill(q: Tensor, k: Tensor, cos: Tensor, sin: Tensor, seq_len: int, num_heads: int,
                       num_kv_heads: int, head_dim: int, start_pos: int) -> None:
    """src/cuda_kernels.rs:670-700."""
    _lib().nve_rope_f16_prefill(_ptr(q, _F16), _ptr(k, _F16), _ptr(cos, _F16), _ptr(sin, _F16), seq_len, num_heads,
                                num_kv_heads, head_dim, start_pos, stream())
    _ffi.check_last("nve_rope_f16_prefill")


def rms_norm_rows(x: Tensor, weight: Tensor, eps: float, out: Optional[Tensor] = None) -> Tensor:
    """RMSNorm of every row of x [rows, n] in one launch (each row as rms_norm computes it)."""
    if x.dim() != 2:
        raise ValueError("x must be [rows, n]")
    out = torch.empty_like(x) if out is None else out
    _ffi.check("nve_b200_rms_norm_rows",
               _lib().nve_b200_rms_norm_rows(_ptr(x, (torch.float16, torch.bfloat16), "x"), _ptr(weight, x.dtype),
                                             _ptr(out, x.dtype), x.shape[0], x.shape[1], float(eps), _dt(x), stream()))
    return out


def add_rms_norm_rows(x: Tensor, delta: Tensor, weight: Tensor, eps: float, out: Optional[Tensor] = None) -> Tensor:
    """x += delta in place, then RMSNorm of every row of x into `out` (returned): add_inplace_any + rms_norm_rows in one
    launch, same bits."""
    if x.dim() != 2 or delta.shape != x.shape:
        raise ValueError("x and delta must be [rows, n]")
    out = torch.empty_like(x) if out is None else out
    _ffi.check("nve_b200_add_rms_norm_rows",
               _lib().nve_b200_add_rms_norm_rows(_ptr(x, (torch.float16, torch.bfloat16), "x"), _ptr(delta, x.dtype),
                                                 _ptr(weight, x.dtype), _ptr(out, x.dtype), x.shape[0], x.shape[1], float(eps),
                                                 _dt(x), stream()))
    return out


def kv_cache_write_rows(k_new: Tensor, k_cache: Tensor, v_new: Tensor, v_cache: Tensor, start_pos: int, num_kv_heads: int,
                        head_dim: int, max_seq_len: int) -> None:
    """cache[kvh, start_pos + s, :] = new[s, kvh, :] for the rows of k_new / v_new [S, nkv, hd]."""
    rows = k_new.shape[0]
    _ffi.check("nve_b200_kv_cache_write_rows",
               _lib().nve_b200_kv_cache_write_rows(_ptr(k_new, _F16, "k_new"), _ptr(k_cache, _F16), _ptr(v_new, _F16, "v_new"),
                                                   _ptr(v_cache, _F16), rows, start_pos, num_kv_heads, head_dim, max_seq_len,
                                                   stream()))


def attn_prefill_causal(q: Tensor, k_cache: Tensor, v_cache: Tensor, start_pos: int, num_heads: int, num_kv_heads: int,
                        head_dim: int, max_seq_len: int, scale: float, out: Optional[Tensor] = None) -> Tensor:
    """Row r of q [S, nh*hd] attends to cache positions [0, start_pos + r]; returns [S, nh*hd]."""
    out = torch.empty_like(q) if out is None else out
    _ffi.check("nve_b200_attn_prefill_causal",
               _lib().nve_b200_attn_prefill_causal(_ptr(q, _F16, "q"), _ptr(k_cache, _F16), _ptr(v_cache, _F16),
                                                   _ptr(out, _F16, "out"), q.shape[0], start_pos, num_heads, num_kv_heads,
                                                   head_dim, max_seq_len, float(scale), stream()))
    return out


def fused_matvec(x: Tensor, w: Tensor, n: int, k: int) -> Tensor:
    """src/cuda_kernels.rs:441-457: dense f16 GEMV, returns [1, n]."""
    out = torch.empty((1, n), dtype=_F16, device=x.device)
    fused_matvec_into(x, w, out, n, k)
    return out


def fused_matvec_into(x: Tensor, w: Tensor, out: Tensor, n: int, k: int) -> None:
    """src/cuda_kernels.rs:717-725."""
    _lib().nve_matvec_f16(_ptr(x, _F16), _ptr(w, _F16), _ptr(out, _F16), n, k, stream())
    _ffi.check_last("nve_matvec_f16")


def fused_matvec_w4a16(x: Tensor, nibbles: Tensor, scales: Tensor, awq_scales: Optional[Tensor], n: int,
                       k: int) -> Tensor:
    """src/cuda_kernels.rs:463-486: returns [1, n] f16."""
    out = torch.empty((1, n), dtype=_F16, device=x.device)
    fused_matvec_w4a16_into(x, nibbles, scales, awq_scales, out, n, k)
    return out


def fused_matvec_w4a16_into(x: Tensor, nibbles: Tensor, scales: Tensor, awq_scales: Optional[Tensor], out: Tensor,
                            n: int, k: int) -> None:
    """src/cuda_kernels.rs:727-745."""
    _lib().nve_matvec_w4a16(_ptr(x, _F16, "x"), _ptr(nibbles, torch.uint8, "nibbles"),
                            _ptr(scales, torch.float32, "scales"), _ptr(awq_scales, torch.float32, "awq"),
                            _ptr(out, _F16, "out"), n, k, stream())
    _ffi.check_last("nve_matvec_w4a16")


def dequant_w4a16(nibbles: Tensor, scales: Tensor, awq_scales: Optional[Tensor], n: int, k: int) -> Tensor:
    """src/cuda_kernels.rs:494-519: full f16 weight matrix [n, k]."""
    out = torch.empty((n, k), dtype=_F16, device=nibbles.device)
    _lib().nve_dequant_w4a16(_ptr(nibbles, torch.uint8), _ptr(scales, torch.float32),
                             _ptr(awq_scales, torch.float32), _ptr(out), n, k, stream())
    _ffi.check_last("nve_dequant_w4a16")
    return out


def quantize_f16_q8(x: Tensor) -> Tuple[Tensor, Tensor]:
    """src/cuda_kernels.rs:525-540: returns (xq [K] int8, xq_scales [K/32] f32)."""
    k = x.numel()
    if k % 32 != 0:
        raise ValueError("quantize_f16_q8: K must be multiple of 32")
    xq = torch.empty(k, dtype=torch.int8, device=x.device)
    scales = torch.empty(k // 32, dtype=torch.float32, device=x.device)
    _lib().nve_quantize_f16_q8(_ptr(x, _F16, "x"), _ptr(xq), _ptr(scales), k, stream())
    _ffi.check_last("nve_quantize_f16_q8")
    return xq, scales


def matvec_w4a8(xq: Tensor, xq_scales: Tensor, nibbles: Tensor, wt_scales: Tensor, n: int, k: int) -> Tensor:
    """src/cuda_kernels.rs:552-573: returns [1, n] f16."""
    out = torch.empty((1, n), dtype=_F16, device=xq.device)
    _lib().nve_matvec_w4a8(_ptr(xq, _Q8, "xq"), _ptr(xq_scales, torch.float32, "xq_scales"),
                           _ptr(nibbles, torch.uint8, "nibbles"), _ptr(wt_scales, torch.float32, "wt_scales"),
                           _ptr(out), n, k, stream())
    _ffi.check_last("nve_matvec_w4a8")
    return out


def flash_decode_f16(q: Tensor, k_cache: Tensor, v_cache: Tensor, num_heads: int, num_kv_heads: int,
                     scale: float) -> Tensor:
    """src/cuda_kernels.rs:586-616: q [nh,hd], caches [nkv,seq,hd] -> [nh,hd]."""
    head_dim = q.shape[1]
    seq_len = k_cache.shape[1]
    out = torch.empty((num_heads, head_dim), dtype=_F16, device=q.device)
    _lib().nve_flash_decode_f16(_ptr(q, _F16, "q"), _ptr(k_cache, _F16, "k_cache"), _ptr(v_cache, _F16, "v_cache"),
                                _ptr(out), num_heads, num_kv_heads, seq_len, head_dim, float(scale), stream())
    _ffi.check_last("nve_flash_decode_f16")
    return out


def fused_qkv_matvec_w4a16(x, q_nib, q_sc, q_awq, nq, k_nib, k_sc, k_awq, nk, v_nib, v_sc, v_awq, nv, k_dim):
    """src/cuda_kernels.rs:622-662: returns ([1,nq], [1,nk], [1,nv]) f16."""
    dev = x.device
    q_out = torch.empty((1, nq), dtype=_F16, device=dev)
    k_out = torch.empty((1, nk), dtype=_F16, device=dev)
    v_out = torch.empty((1, nv), dtype=_F16, device=dev)
    fused_qkv_matvec_w4a16_into(x, q_nib, q_sc, q_awq, nq, k_nib, k_sc, k_awq, nk, v_nib, v_sc, v_awq, nv, q_out,
                                k_out, v_out, k_dim)
    return q_out, k_out, v_out


def fused_qkv_matvec_w4a16_into(x, q_nib, q_sc, q_awq, nq, k_nib, k_sc, k_awq, nk, v_nib, v_sc, v_awq, nv, q_out,
                                k_out, v_out, k_dim) -> None:
    """src/cuda_kernels.rs:749-786."""
    u8, f32 = torch.uint8, torch.float32
    _lib().nve_qkv_matvec_w4a16(_ptr(x, _F16, "x"), _ptr(q_nib, u8), _ptr(q_sc, f32), _ptr(q_awq, f32), nq,
                                _ptr(k_nib, u8), _ptr(k_sc, f32), _ptr(k_awq, f32), nk, _ptr(v_nib, u8),
                                _ptr(v_sc, f32), _ptr(v_awq, f32), nv, _ptr(q_out, _F16), _ptr(k_out, _F16),
                                _ptr(v_out, _F16), k_dim, stream())
    _ffi.check_last("nve_qkv_matvec_w4a16")


def kv_cache_write(k_new: Tensor, k_cache: Tensor, v_new: Tensor, v_cache: Tensor, d_pos: int, num_kv_heads: int,
                   head_dim: int, max_seq_len: int) -> None:
    """src/cuda_kernels.rs:793-816: d_pos is a device address of an int (e.g. graph_d_pos_ptr())."""
    _lib().nve_kv_cache_write_f16(_ptr(k_new, _F16), _ptr(k_cache, _F16), _ptr(v_new, _F16), _ptr(v_cache, _F16),
                                  d_pos, num_kv_heads, head_dim, max_seq_len, stream())
    _ffi.check_last("nve_kv_cache_write_f16")


def add_inplace(dst: Tensor, src: Tensor) -> None:
    """src/cuda_kernels.rs:818-825."""
    _lib().nve_add_inplace_f16(_ptr(dst, _F16), _ptr(src, _F16), dst.numel(), stream())
    _ffi.check_last("nve_add_inplace_f16")


def silu_mul_inplace(gate: Tensor, up: Tensor) -> None:
    """src/cuda_kernels.rs:827-835."""
    _lib().nve_silu_mul_f16(_ptr(gate, _F16), _ptr(up, _F16), gate.numel(), stream())
    _ffi.check_last("nve_silu_mul_f16")


def rope_decode_dyn_inplace(q: Tensor, k: Tensor, cos_tab: Tensor, sin_tab: Tensor, num_heads: int,
                            num_kv_heads: int, head_dim: int, d_pos: int) -> None:
    """src/cuda_kernels.rs:837-862."""
    _lib().nve_rope_f16_decode_dyn(_ptr(q, _F16), _ptr(k, _F16), _ptr(cos_tab, _F16), _ptr(sin_tab, _F16), num_heads,
                                   num_kv_heads, head_dim, d_pos, stream())
    _ffi.check_last("nve_rope_f16_decode_dyn")


def flash_decode_dyn_into(q: Tensor, k_cache: Tensor, v_cache: Tensor, out: Tensor, num_heads: int,
                          num_kv_heads: int, d_seq_len: int, head_dim: int, scale: float, max_seq_len: int) -> None:
    """src/cuda_kernels.rs:864-890."""
    _lib().nve_flash_decode_dyn(_ptr(q, _F16), _ptr(k_cache, _F16), _ptr(v_cache, _F16), _ptr(out, _F16), num_heads,
                                num_kv_heads, d_seq_len, head_dim, float(scale), max_seq_len, stream())
    _ffi.check_last("nve_flash_decode_dyn")


def device_copy(dst: Tensor, src: Tensor) -> None:
    """src/cuda_kernels.rs:892-901."""
    nbytes = src.numel() * src.element_size()
    if dst.numel() * dst.element_size() < nbytes:
        raise ValueError("device_copy: destination too small")
    _lib().nve_d2d_copy(_ptr(dst), _ptr(src), nbytes, stream())
    _ffi.check_last("nve_d2d_copy")


def graph_init() -> None:
    """src/cuda_kernels.rs:903-907."""
    _lib().nve_graph_init()
    _ffi.check_last("nve_graph_init")


def graph_begin_capture() -> None:
    """src/cuda_kernels.rs:909-914: opens capture and routes this thread's launches to the capture stream."""
    lib = _lib()
    lib.nve_graph_begin_capture()
    _ffi.check_last("nve_graph_begin_capture")
    set_graph_capture_stream(lib.nve_graph_capture_stream())


def graph_end_capture() -> None:
    """src/cuda_kernels.rs:916-920."""
    clear_graph_capture_stream()
    _lib().nve_graph_end_capture()
    _ffi.check_last("nve_graph_end_capture")


def graph_launch(pos: int, seq_len: int, on_stream: Optional[int] = None) -> None:
    """src/cuda_kernels.rs:922-925 (the Rust side always launches on the legacy default stream)."""
    _lib().nve_graph_launch(int(pos), int(seq_len), stream() if on_stream is None else on_stream)
    _ffi.check_last("nve_graph_launch")


def graph_ready() -> bool:
    """src/cuda_kernels.rs:927-930."""
    return _lib().nve_graph_ready() != 0


def graph_destroy() -> None:
    """src/cuda_kernels.rs:932-935."""
    clear_graph_capture_stream()
    _lib().nve_graph_destroy()


def graph_d_pos_ptr() -> int:
    """src/cuda_kernels.rs:937-940."""
    return _lib().nve_graph_d_pos()


def graph_d_seqlen_ptr() -> int:
    """src/cuda_kernels.rs:942-945."""
    return _lib().nve_graph_d_seqlen()


# --------------------------------------------------------------------------- additive wrappers
def launch_count() -> int:
    return int(_lib().nve_b200_launch_count())


def set_pdl(enabled: bool) -> bool:
    return bool(_lib().nve_b200_set_pdl(int(enabled)))


def set_attn_decode_kernel(cuda_core: bool) -> bool:
    """Which kernel attn_decode_fused launches: the tensor-core kernel (default) or, with cuda_core=True, the CUDA-core
    kernel whose results equal the un-fused launch sequence bit for bit.  Returns the previous setting."""
    return bool(_lib().nve_b200_set_attn_decode_kernel(1 if cuda_core else 0))


@contextlib.contextmanager
def attn_decode_kernel(cuda_core: bool):
    """`with attn_decode_kernel(True): ...` runs (or captures) the block with the CUDA-core decode attention."""
    prev = set_attn_decode_kernel(cuda_core)
    try:
        yield
    finally:
        set_attn_decode_kernel(prev)


def quantize_q8(x: Tensor) -> Tuple[Tensor, Tensor]:
    """quantize_f16_q8 for f16 or bf16 activations."""
    k = x.numel()
    if k % 32 != 0:
        raise ValueError("quantize_q8: K must be multiple of 32")
    xq = torch.empty(k, dtype=torch.int8, device=x.device)
    scales = torch.empty(k // 32, dtype=torch.float32, device=x.device)
    _ffi.check("nve_b200_quantize_q8", _lib().nve_b200_quantize_q8(_ptr(x, (torch.float16, torch.bfloat16)), _ptr(xq),
                                                                   _ptr(scales), k, _dt(x), stream()))
    return xq, scales


def quantize_q8_awq(x: Tensor, awq_inv: Tensor) -> Tuple[Tensor, Tensor]:
    """int8 codes of x * awq_inv (per column), per group of 32: the W4A8 quantiser for AWQ pre-scaled weights."""
    k = x.numel()
    xq = torch.empty(k, dtype=torch.int8, device=x.device)
    scales = torch.empty(k // 32, dtype=torch.float32, device=x.device)
    _ffi.check("nve_b200_quantize_q8_awq",
               _lib().nve_b200_quantize_q8_awq(_ptr(x, (torch.float16, torch.bfloat16), "x"), _ptr(awq_inv, torch.float32),
                                               _ptr(xq), _ptr(scales), k, _dt(x), stream()))
    return xq, scales


def rms_norm(x: Tensor, weight: Tensor, eps: float, out: Optional[Tensor] = None) -> Tensor:
    out = torch.empty_like(x) if out is None else out
    _ffi.check("nve_b200_rms_norm", _lib().nve_b200_rms_norm(_ptr(x), _ptr(weight, x.dtype), _ptr(out, x.dtype),
                                                             x.numel(), float(eps), _dt(x), stream()))
    return out


def rmsnorm_quantize_q8(x: Tensor, weight: Tensor, eps: float, want_normed: bool = False, xq: Optional[Tensor] = None,
                        scales: Optional[Tensor] = None, normed: Optional[Tensor] = None):
    """RMSNorm -> 16-bit round -> int8 quantisation in one launch; returns (xq, scales, normed|None)."""
    n = x.numel()
    xq = torch.empty(n, dtype=torch.int8, device=x.device) if xq is None else xq
    scales = torch.empty(n // 32, dtype=torch.float32, device=x.device) if scales is None else scales
    if normed is None and want_normed:
        normed = torch.empty_like(x)
    _ffi.check("nve_b200_rmsnorm_quantize_q8",
               _lib().nve_b200_rmsnorm_quantize_q8(_ptr(x), _ptr(weight, x.dtype), _ptr(normed, x.dtype), _ptr(xq, _Q8),
                                                   _ptr(scales, torch.float32), n, float(eps), _dt(x), stream()))
    return xq, scales, normed


def silu_mul_quantize_q8(gate: Tensor, up: Tensor, want_mid: bool = False, xq: Optional[Tensor] = None,
                         scales: Optional[Tensor] = None, mid: Optional[Tensor] = None):
    """silu(gate)*up -> 16-bit round -> int8 quantisation in one launch; returns (xq, scales, mid|None)."""
    n = gate.numel()
    xq = torch.empty(n, dtype=torch.int8, device=gate.device) if xq is None else xq
    scales = torch.empty(n // 32, dtype=torch.float32, device=gate.device) if scales is None else scales
    if mid is None and want_mid:
        mid = torch.empty_like(gate)
    _ffi.check("nve_b200_silu_mul_quantize_q8",
               _lib().nve_b200_silu_mul_quantize_q8(_ptr(gate), _ptr(up, gate.dtype), _ptr(mid, gate.dtype),
                                                    _ptr(xq, _Q8), _ptr(scales, torch.float32), n, _dt(gate), stream()))
    return xq, scales, mid


def silu_mul_x16(gate: Tensor, up: Tensor, awq: Optional[Tensor] = None, want_mid: bool = False,
                 x_lo: Optional[Tensor] = None, x_hi: Optional[Tensor] = None, scales: Optional[Tensor] = None,
                 mid: Optional[Tensor] = None):
    """silu(gate)*up -> 16-bit round -> [* awq] -> 16-bit fixed-point byte planes for the W4A16 GEMV, one launch;
    returns (x_lo uint8 [n], x_hi int8 [n], scales f32 [n/32], mid|None)."""
    n = gate.numel()
    dev = gate.device
    x_lo = torch.empty(n, dtype=torch.uint8, device=dev) if x_lo is None else x_lo
    x_hi = torch.empty(n, dtype=torch.int8, device=dev) if x_hi is None else x_hi
    scales = torch.empty(n // 32, dtype=torch.float32, device=dev) if scales is None else scales
    if mid is None and want_mid:
        mid = torch.empty_like(gate)
    _ffi.check("nve_b200_silu_mul_x16",
               _lib().nve_b200_silu_mul_x16(_ptr(gate), _ptr(up, gate.dtype), _ptr(mid, gate.dtype), _ptr(x_lo, torch.uint8),
                                            _ptr(x_hi, _Q8), _ptr(scales, torch.float32), _ptr(awq, torch.float32), n,
                                            _dt(gate), stream()))
    return x_lo, x_hi, scales, mid


def silu_mul(gate: Tensor, up: Tensor) -> None:
    _ffi.check("nve_b200_silu_mul", _lib().nve_b200_silu_mul(_ptr(gate), _ptr(up, gate.dtype), gate.numel(), _dt(gate),
                                                             stream()))


def add_inplace_any(dst: Tensor, src: Tensor) -> None:
    _ffi.check("nve_b200_add_inplace", _lib().nve_b200_add_inplace(_ptr(dst), _ptr(src, dst.dtype), dst.numel(),
                                                                   _dt(dst), stream()))


def _mats(weights: Sequence, outs: Sequence[Tensor], residuals: Optional[Sequence[Optional[Tensor]]], out_dtype):
    arr = (W4Matrix * len(weights))()
    for i, (w, o) in enumerate(zip(weights, outs)):
        nib, sc, n = w
        r = residuals[i] if residuals is not None else None
        arr[i] = W4Matrix(_ptr(nib, torch.uint8, "nibbles"), _ptr(sc, torch.float32, "scales"), _ptr(o, out_dtype, "out"),
                          _ptr(r, out_dtype, "residual"), int(n))
    return arr


def matvec_w4a8_multi(xq: Tensor, xq_scales: Tensor, weights: Sequence, k: int, out_dtype=torch.float16,
                      outs: Optional[Sequence[Tensor]] = None, residuals=None):
    """W4A8 GEMV over 1..3 matrices sharing the activation codes.  weights: [(nibbles, scales, n), ...]."""
    if outs is None:
        outs = [torch.empty((1, n), dtype=out_dtype, device=xq.device) for (_, _, n) in weights]
    arr = _mats(weights, outs, residuals, out_dtype)
    _ffi.check("nve_b200_matvec_w4a8_multi",
               _lib().nve_b200_matvec_w4a8_multi(_ptr(xq, _Q8, "xq"), _ptr(xq_scales, torch.float32), arr, len(weights), k,
                                                 _TORCH_DT[out_dtype], stream()))
    return list(outs)


def matvec_w4a16_multi(x: Tensor, awq: Optional[Tensor], weights: Sequence, k: int, out_dtype=torch.float16,
                       outs: Optional[Sequence[Tensor]] = None, residuals=None):
    """W4A16 GEMV over 1..3 matrices sharing x (f16 or bf16) and the optional awq vector."""
    if outs is None:
        outs = [torch.empty((1, n), dtype=out_dtype, device=x.device) for (_, _, n) in weights]
    arr = _mats(weights, outs, residuals, out_dtype)
    _ffi.check("nve_b200_matvec_w4a16_multi",
               _lib().nve_b200_matvec_w4a16_multi(_ptr(x, (torch.float16, torch.bfloat16), "x"), _dt(x),
                                                  _ptr(awq, torch.float32), arr, len(weights), k, _TORCH_DT[out_dtype],
                                                  stream()))
    return list(outs)


def matvec_w4a16_planes_multi(x_lo: Tensor, x_hi: Tensor, x_scales: Tensor, weights: Sequence, k: int,
                              out_dtype=torch.float16, outs: Optional[Sequence[Tensor]] = None, residuals=None):
    """W4A16 GEMV over 1..3 matrices from activations already in fixed-point plane form (silu_mul_x16)."""
    if outs is None:
        outs = [torch.empty((1, n), dtype=out_dtype, device=x_lo.device) for (_, _, n) in weights]
    arr = _mats(weights, outs, residuals, out_dtype)
    _ffi.check("nve_b200_matvec_w4a16_planes_multi",
               _lib().nve_b200_matvec_w4a16_planes_multi(_ptr(x_lo, torch.uint8), _ptr(x_hi, _Q8),
                                                         _ptr(x_scales, torch.float32), arr, len(weights), k,
                                                         _TORCH_DT[out_dtype], stream()))
    return list(outs)


def rmsnorm_matvec_w4a8_multi(h: Tensor, norm_weight: Tensor, eps: float, weights: Sequence, k: int,
                              out_dtype=torch.float16, outs: Optional[Sequence[Tensor]] = None, residuals=None):
    """RMSNorm -> int8 quantise -> W4A8 GEMV over 1..3 matrices, one launch (bit-identical to the separate calls)."""
    if outs is None:
        outs = [torch.empty((1, n), dtype=out_dtype, device=h.device) for (_, _, n) in weights]
    arr = _mats(weights, outs, residuals, out_dtype)
    _ffi.check("nve_b200_rmsnorm_matvec_w4a8_multi",
               _lib().nve_b200_rmsnorm_matvec_w4a8_multi(_ptr(h, (torch.float16, torch.bfloat16), "h"),
                                                         _ptr(norm_weight, h.dtype, "norm_weight"), float(eps), _dt(h), arr,
                                                         len(weights), k, _TORCH_DT[out_dtype], stream()))
    return list(outs)


def rmsnorm_matvec_w4a8_awq_multi(h: Tensor, norm_weight: Tensor, eps: float, awq_inv: Tensor, weights: Sequence, k: int,
                                  out_dtype=torch.float16, outs: Optional[Sequence[Tensor]] = None, residuals=None):
    """rmsnorm_matvec_w4a8_multi with the AWQ multiplier folded into the activation quantiser."""
    if outs is None:
        outs = [torch.empty((1, n), dtype=out_dtype, device=h.device) for (_, _, n) in weights]
    arr = _mats(weights, outs, residuals, out_dtype)
    _ffi.check("nve_b200_rmsnorm_matvec_w4a8_awq_multi",
               _lib().nve_b200_rmsnorm_matvec_w4a8_awq_multi(_ptr(h, (torch.float16, torch.bfloat16), "h"),
                                                             _ptr(norm_weight, h.dtype, "norm_weight"), float(eps), _dt(h),
                                                             _ptr(awq_inv, torch.float32), arr, len(weights), k,
                                                             _TORCH_DT[out_dtype], stream()))
    return list(outs)


def rmsnorm_matvec_w4a16_multi(h: Tensor, norm_weight: Tensor, eps: float, awq: Optional[Tensor], weights: Sequence,
                               k: int, out_dtype=torch.float16, outs: Optional[Sequence[Tensor]] = None, residuals=None):
    """RMSNorm -> W4A16 GEMV over 1..3 matrices, one launch (bit-identical to the separate calls)."""
    if outs is None:
        outs = [torch.empty((1, n), dtype=out_dtype, device=h.device) for (_, _, n) in weights]
    arr = _mats(weights, outs, residuals, out_dtype)
    _ffi.check("nve_b200_rmsnorm_matvec_w4a16_multi",
               _lib().nve_b200_rmsnorm_matvec_w4a16_multi(_ptr(h, (torch.float16, torch.bfloat16), "h"),
                                                          _ptr(norm_weight, h.dtype, "norm_weight"), float(eps), _dt(h),
                                                          _ptr(awq, torch.float32), arr, len(weights), k,
                                                          _TORCH_DT[out_dtype], stream()))
    return list(outs)


def rmsnorm_gateup_silu(h: Tensor, norm_weight: Tensor, eps: float, awq: Optional[Tensor], gate, up, k: int, use_w4a8: bool,
                        mid: Optional[Tensor] = None, quant: Optional[dict] = None) -> Tensor:
    """RMSNorm + gate/up GEMV + SiLU*up in one launch; gate / up are (nibbles, scales, n) triples; returns mid [1, n].

    `quant` also leaves mid converted for the down projection (the CTA that completes a 32-wide group converts it):
    W4A8 route {"xq": int8 [n], "xs": f32 [n/32], "counters": int32 [n/32]}; W4A16 route {"xlo": uint8 [n], "xhi": int8
    [n], "xs": ..., "counters": ..., "down_awq": optional f32 [n]}.  `counters` is zeroed once by the caller and then
    only ever passed to launches for this mid vector."""
    n = gate[2]
    mid = torch.empty((1, n), dtype=h.dtype, device=h.device) if mid is None else mid
    g = W4Matrix(_ptr(gate[0], torch.uint8), _ptr(gate[1], torch.float32), None, None, n)
    u = W4Matrix(_ptr(up[0], torch.uint8), _ptr(up[1], torch.float32), None, None, up[2])
    head = (_ptr(h, (torch.float16, torch.bfloat16), "h"), _ptr(norm_weight, h.dtype), float(eps), _dt(h),
            _ptr(awq, torch.float32), C.byref(g), C.byref(u), _ptr(mid, h.dtype), k)
    if quant is None:
        fn = "nve_b200_rmsnorm_gateup_silu_w4a8" if use_w4a8 else "nve_b200_rmsnorm_gateup_silu_w4a16"
        _ffi.check(fn, getattr(_lib(), fn)(*head, stream()))
    elif use_w4a8:
        fn = "nve_b200_rmsnorm_gateup_silu_q8_w4a8"
        _ffi.check(fn, getattr(_lib(), fn)(*head, _ptr(quant["xq"], _Q8, "xq"), _ptr(quant["xs"], torch.float32, "xs"),
                                           _ptr(quant["counters"], torch.int32, "counters"), stream()))
    else:
        fn = "nve_b200_rmsnorm_gateup_silu_x16_w4a16"
        _ffi.check(fn, getattr(_lib(), fn)(*head, _ptr(quant["xlo"], torch.uint8, "xlo"), _ptr(quant["xhi"], _Q8, "xhi"),
                                           _ptr(quant["xs"], torch.float32, "xs"), _ptr(quant.get("down_awq"), torch.float32),
                                           _ptr(quant["counters"], torch.int32, "counters"), stream()))
    return mid


def quantize_matvec_w4a8_multi(x: Tensor, awq_inv: Optional[Tensor], weights: Sequence, k: int,
                               outs: Optional[Sequence[Tensor]] = None, residuals=None, allreduce: bool = False):
    """int8 quantisation of the 16-bit vector x in the GEMV prologue + W4A8 GEMV (outputs of x's type)."""
    if outs is None:
        outs = [torch.empty((1, n), dtype=x.dtype, device=x.device) for (_, _, n) in weights]
    arr = _mats(weights, outs, residuals, x.dtype)
    if allreduce:
        _ffi.check("nve_b200_quantize_matvec_w4a8_allreduce",
                   _lib().nve_b200_quantize_matvec_w4a8_allreduce(_ptr(x, (torch.float16, torch.bfloat16), "x"), _dt(x),
                                                                  _ptr(awq_inv, torch.float32), arr, k, stream()))
    else:
        _ffi.check("nve_b200_quantize_matvec_w4a8_multi",
                   _lib().nve_b200_quantize_matvec_w4a8_multi(_ptr(x, (torch.float16, torch.bfloat16), "x"), _dt(x),
                                                              _ptr(awq_inv, torch.float32), arr, len(weights), k, stream()))
    return list(outs)


def attn_decode_fused(q: Tensor, k_new: Tensor, v_new: Tensor, k_cache: Tensor, v_cache: Tensor, cos_tab: Tensor,
                      sin_tab: Tensor, d_pos: int, d_seq_len: int, out: Tensor, num_heads: int, num_kv_heads: int,
                      head_dim: int, max_seq_len: int, scale: float, out_q: Optional[Tensor] = None,
                      out_scales: Optional[Tensor] = None) -> None:
    """RoPE + KV-cache write + flash decode (+ int8 quantisation of the output) in one launch."""
    _ffi.check("nve_b200_attn_decode_fused",
               _lib().nve_b200_attn_decode_fused(_ptr(q, _F16, "q"), _ptr(k_new, _F16, "k_new"), _ptr(v_new, _F16, "v_new"),
                                                 _ptr(k_cache, _F16), _ptr(v_cache, _F16), _ptr(cos_tab, _F16),
                                                 _ptr(sin_tab, _F16), d_pos, d_seq_len, _ptr(out, _F16, "out"),
                                                 _ptr(out_q, _Q8), _ptr(out_scales, torch.float32), num_heads,
                                                 num_kv_heads, head_dim, max_seq_len, float(scale), stream()))


def attn_decode_fused_batch(q: Tensor, k_new: Tensor, v_new: Tensor, k_cache: Tensor, v_cache: Tensor, cos_tab: Tensor,
                            sin_tab: Tensor, d_pos: Tensor, d_seq_len: Tensor, num_heads: int, num_kv_heads: int,
                            head_dim: int, max_seq_len: int, scale: float, out: Optional[Tensor] = None) -> Tensor:
    """attn_decode_fused for B independent sequences in one launch: q [B, nh*hd], k_new / v_new [B, nkv*hd], caches
    [B, nkv, max_seq, hd], d_pos / d_seq_len int32 [B] on the device; returns [B, nh*hd]."""
    b = q.shape[0]
    if k_cache.shape[0] != b or d_pos.numel() != b or d_seq_len.numel() != b:
        raise ValueError("one cache, position and length per row of q")
    out = torch.empty_like(q) if out is None else out
    _ffi.check("nve_b200_attn_decode_fused_batch",
               _lib().nve_b200_attn_decode_fused_batch(
                   _ptr(q, _F16, "q"), _ptr(k_new, _F16, "k_new"), _ptr(v_new, _F16, "v_new"), _ptr(k_cache, _F16),
                   _ptr(v_cache, _F16), _ptr(cos_tab, _F16), _ptr(sin_tab, _F16), _ptr(d_pos, torch.int32, "d_pos"),
                   _ptr(d_seq_len, torch.int32, "d_seq_len"), _ptr(out, _F16, "out"), b, num_heads, num_kv_heads, head_dim,
                   max_seq_len, float(scale), stream()))
    return out


# --------------------------------------------------------------------------- whole step in one kernel
def decode_step_workspace_bytes(model: "_ffi.DecodeModel") -> int:
    n = int(_lib().nve_b200_decode_step_workspace_bytes(C.byref(model)))
    _ffi.check_last("nve_b200_decode_step_workspace_bytes")
    return n


def decode_step_init(workspace: Tensor) -> None:
    _ffi.check("nve_b200_decode_step_init",
               _lib().nve_b200_decode_step_init(_ptr(workspace), workspace.numel() * workspace.element_size(), stream()))


def decode_step(model: "_ffi.DecodeModel", layers_dev: Tensor, hidden: Tensor, d_pos: int, d_seqlen: int,
                workspace: Tensor) -> None:
    """One token through all layers in one persistent kernel (nve_b200_decode_step); `hidden` is updated in place."""
    _ffi.check("nve_b200_decode_step",
               _lib().nve_b200_decode_step(C.byref(model), _ptr(layers_dev), _ptr(hidden, _F16, "hidden"), d_pos, d_seqlen,
                                           _ptr(workspace), workspace.numel() * workspace.element_size(), stream()))


def decode_step_error(workspace: Tensor, reset: bool = False) -> int:
    return int(_lib().nve_b200_decode_step_error(_ptr(workspace), int(reset)))


def decode_step_set_prefetch(nbytes: int) -> int:
    return int(_lib().nve_b200_decode_step_set_prefetch(int(nbytes)))


def decode_step_wait_probe(workspace: Tensor, wait_ns: int) -> None:
    _ffi.check("nve_b200_decode_step_wait_probe", _lib().nve_b200_decode_step_wait_probe(_ptr(workspace), int(wait_ns), stream()))


def matvec_w4a8_allreduce(xq: Tensor, xq_scales: Tensor, weights: Sequence, k: int, out_dtype=torch.float16,
                          outs: Optional[Sequence[Tensor]] = None, residuals=None):
    """Row-parallel W4A8 GEMV of one matrix with the all-reduce over the tensor-parallel ranks fused in."""
    if len(weights) != 1:
        raise ValueError("the fused all-reduce takes one matrix")
    if outs is None:
        outs = [torch.empty((1, weights[0][2]), dtype=out_dtype, device=xq.device)]
    arr = _mats(weights, outs, residuals, out_dtype)
    _ffi.check("nve_b200_matvec_w4a8_allreduce",
               _lib().nve_b200_matvec_w4a8_allreduce(_ptr(xq, _Q8, "xq"), _ptr(xq_scales, torch.float32), arr, k,
                                                     _TORCH_DT[out_dtype], stream()))
    return list(outs)


def matvec_w4a16_allreduce(x: Tensor, awq: Optional[Tensor], weights: Sequence, k: int, out_dtype=torch.float16,
                           outs: Optional[Sequence[Tensor]] = None, residuals=None):
    """Row-parallel W4A16 GEMV of one matrix with the all-reduce over the tensor-parallel ranks fused in."""
    if len(weights) != 1:
        raise ValueError("the fused all-reduce takes one matrix")
    if outs is None:
        outs = [torch.empty((1, weights[0][2]), dtype=out_dtype, device=x.device)]
    arr = _mats(weights, outs, residuals, out_dtype)
    _ffi.check("nve_b200_matvec_w4a16_allreduce",
               _lib().nve_b200_matvec_w4a16_allreduce(_ptr(x, (torch.float16, torch.bfloat16), "x"), _dt(x),
                                                      _ptr(awq, torch.float32), arr, k, _TORCH_DT[out_dtype], stream()))
    return list(outs)


def matvec_w4a16_planes_allreduce(x_lo: Tensor, x_hi: Tensor, x_scales: Tensor, weights: Sequence, k: int,
                                  out_dtype=torch.float16, outs: Optional[Sequence[Tensor]] = None, residuals=None):
    """matvec_w4a16_allreduce fed with the fixed-point planes written by silu_mul_x16."""
    if len(weights) != 1:
        raise ValueError("the fused all-reduce takes one matrix")
    if outs is None:
        outs = [torch.empty((1, weights[0][2]), dtype=out_dtype, device=x_lo.device)]
    arr = _mats(weights, outs, residuals, out_dtype)
    _ffi.check("nve_b200_matvec_w4a16_planes_allreduce",
               _lib().nve_b200_matvec_w4a16_planes_allreduce(_ptr(x_lo, torch.uint8), _ptr(x_hi, _Q8),
                                                             _ptr(x_scales, torch.float32), arr, k, _TORCH_DT[out_dtype],
                                                             stream()))
    return list(outs)


def gemm_w4a16_scratch_bytes(m: int, n: int, k: int) -> int:
    return int(_lib().nve_b200_gemm_w4a16_scratch_bytes(m, n, k))


def gemm_w4a16(x: Tensor, nibbles: Tensor, scales: Tensor, n: int, k: int, out_dtype=None, out: Optional[Tensor] = None,
               scratch: Optional[Tensor] = None) -> Tensor:
    """Batched W4A16 GEMM on the tensor cores: x [M, K] (f16/bf16), M <= 64 -> [M, n].  `scratch` (uint8/float
    tensor of gemm_w4a16_scratch_bytes) lets the CTAs share tiles over K (few tiles fill all SMs, uneven tile counts are balanced); bf16 activations need it for their f16 copy
    (allocated here when not given)."""
    m = x.shape[0]
    out_dtype = x.dtype if out_dtype is None else out_dtype
    out = torch.empty((m, n), dtype=out_dtype, device=x.device) if out is None else out
    if scratch is None and x.dtype == torch.bfloat16:  # the library needs room for an f16 copy of bf16 activations
        scratch = torch.empty(((m * k * 2 + 255) // 256) * 256, dtype=torch.uint8, device=x.device)
    sb = 0 if scratch is None else scratch.numel() * scratch.element_size()
    _ffi.check("nve_b200_gemm_w4a16",
               _lib().nve_b200_gemm_w4a16(_ptr(x, (torch.float16, torch.bfloat16), "x"), _dt(x), _ptr(nibbles, torch.uint8),
                                          _ptr(scales, torch.float32), _ptr(out, out_dtype, "out"), _TORCH_DT[out_dtype], m, n, k,
                                          _ptr(scratch), sb, stream()))
    return out


def gemm_w4a16_multi_scratch_bytes(m: int, ns: Sequence[int], k: int) -> int:
    import ctypes

    arr = (ctypes.c_int * len(ns))(*[int(n) for n in ns])
    return int(_lib().nve_b200_gemm_w4a16_multi_scratch_bytes(m, ctypes.cast(arr, ctypes.c_void_p), len(ns), k))


def gemm_w4a16_multi(x: Tensor, weights: Sequence, k: int, out_dtype=None, outs: Optional[Sequence[Tensor]] = None,
                     scratch: Optional[Tensor] = None):
    """The batched W4A16 GEMM over 1..3 matrices sharing x [M, K] (q/k/v or gate/up) in one launch.
    weights: [(nibbles, scales, n), ...] -> [M, n] each."""
    m = x.shape[0]
    out_dtype = x.dtype if out_dtype is None else out_dtype
    if outs is None:
        outs = [torch.empty((m, n), dtype=out_dtype, device=x.device) for (_, _, n) in weights]
    if scratch is None and x.dtype == torch.bfloat16:
        scratch = torch.empty(((m * k * 2 + 255) // 256) * 256, dtype=torch.uint8, device=x.device)
    sb = 0 if scratch is None else scratch.numel() * scratch.element_size()
    arr = _mats(weights, outs, None, out_dtype)
    _ffi.check("nve_b200_gemm_w4a16_multi",
               _lib().nve_b200_gemm_w4a16_multi(_ptr(x, (torch.float16, torch.bfloat16), "x"), _dt(x), arr, len(weights),
                                                _TORCH_DT[out_dtype], m, k, _ptr(scratch), sb, stream()))
    return list(outs)


def gemm_w4a16_noalloc(x: Tensor, nibbles: Tensor, scales: Tensor, n: int, k: int, out: Tensor) -> Tensor:
    """Batched W4A16 GEMM for callers that cannot allocate: the caller passes input and output tensors only, the
    workspace for partial tiles is a fixed 4 MiB array inside the library (shapes needing more raise NVE_ERR_TOO_LARGE).
    Calls share that array: keep them on one stream.  Make the first call on a device outside stream capture."""
    _ffi.check("nve_b200_gemm_w4a16_noalloc",
               _lib().nve_b200_gemm_w4a16_noalloc(_ptr(x, (torch.float16, torch.bfloat16), "x"), _dt(x),
                                                  _ptr(nibbles, torch.uint8), _ptr(scales, torch.float32), _ptr(out, None, "out"),
                                                  _dt(out), x.shape[0], n, k, stream()))
    return out


def gemm_error(reset: bool = False) -> int:
    return int(_lib().nve_b200_gemm_error(int(reset)))


def w4a8_idot(xq: Tensor, nibbles: Tensor, n: int, k: int) -> Tensor:
    """Exact per-block integer dots I[n, k/32] (int32)."""
    out = torch.empty((n, k // 32), dtype=torch.int32, device=xq.device)
    _ffi.check("nve_b200_w4a8_idot", _lib().nve_b200_w4a8_idot(_ptr(xq, _Q8), _ptr(nibbles, torch.uint8), _ptr(out), n, k,
                                                               stream()))
    return out


def dequant_w4a16_any(nibbles: Tensor, scales: Tensor, awq: Optional[Tensor], n: int, k: int,
                      out_dtype=torch.float16) -> Tensor:
    out = torch.empty((n, k), dtype=out_dtype, device=nibbles.device)
    _ffi.check("nve_b200_dequant_w4a16",
               _lib().nve_b200_dequant_w4a16(_ptr(nibbles, torch.uint8), _ptr(scales, torch.float32),
                                             _ptr(awq, torch.float32), _ptr(out), n, k, _TORCH_DT[out_dtype], stream()))
    return out


def q4_quantize(w: Tensor, awq_scales: Optional[Tensor] = None) -> Tuple[Tensor, Tensor]:
    """On-device Q4 quantisation of an f32 [N,K] matrix -> (nibbles [N,K/2] u8, scales [N,K/32] f32)."""
    n, k = w.shape
    nib = torch.empty((n, k // 2), dtype=torch.uint8, device=w.device)
    sc = torch.empty((n, k // 32), dtype=torch.float32, device=w.device)
    _ffi.check("nve_b200_q4_quantize", _lib().nve_b200_q4_quantize(_ptr(w, torch.float32, "W"),
                                                                   _ptr(awq_scales, torch.float32), _ptr(nib), _ptr(sc),
                                                                   n, k, stream()))
    return nib, sc


def q4_repack_blocks(cpu_blocks: Tensor, n: int, k: int) -> Tuple[Tensor, Tensor]:
    """Reference CPU blocks (uint8 [n*k/32*20], already on the device) -> device layout."""
    nib = torch.empty((n, k // 2), dtype=torch.uint8, device=cpu_blocks.device)
    sc = torch.empty((n, k // 32), dtype=torch.float32, device=cpu_blocks.device)
    _ffi.check("nve_b200_q4_repack_blocks", _lib().nve_b200_q4_repack_blocks(_ptr(cpu_blocks, torch.uint8), _ptr(nib),
                                                                             _ptr(sc), n, k, stream()))
    return nib, sc


def fill_normal(n: int, seed: int, stream_id: int, first: int = 0, scale: float = 1.0, dtype=torch.float32,
                device="cuda", out: Optional[Tensor] = None) -> Tensor:
    """Counter-based synthetic values generated on the device (bit-identical to the host generator)."""
    out = torch.empty(n, dtype=dtype, device=device) if out is None else out
    lib = _lib()
    if out.dtype == torch.float32:
        st = lib.nve_b200_fill_normal(_ptr(out), n, seed, stream_id, first, float(scale), stream())
    else:
        st = lib.nve_b200_fill_normal_16(_ptr(out), n, seed, stream_id, first, float(scale), _dt(out), stream())
    _ffi.check("nve_b200_fill_normal", st)
    return out
