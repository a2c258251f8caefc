"""CPU oracle for the NVE quantized decode path -- TEST INFRASTRUCTURE ONLY.

ctypes front-end over ``liboracle.so`` (built from ``nve_oracle.c`` by the Makefile
in this directory).  Nothing in the product package may import this module; only the
test suite, the smoke check and the benchmark's CPU-baseline leg do.

Every wrapper takes and returns numpy arrays; docstrings name the C function and,
through it, the reference file:line it restates.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile liboracle.so with the Makefile beside this file (gcc only)."""
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(
        os.path.join(_HERE, "nve_oracle.c")
    ):
        subprocess.check_call(["make", "-B", "-C", _HERE, "liboracle.so"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.orc_have_avx2.restype = C.c_int
        _lib.orc_get_threads.restype = C.c_int
        _lib.orc_use_w4a8.restype = C.c_int
        _lib.orc_use_w4a8.argtypes = [C.c_double, C.c_double, C.c_int]
    return _lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _c(a, dtype) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=dtype)


def _l(v) -> C.c_long:
    return C.c_long(int(v))


# --------------------------------------------------------------------------- 16-bit helpers
def f32_to_f16_bits(x) -> np.ndarray:
    x = _c(x, np.float32)
    out = np.empty(x.shape, np.uint16)
    lib().orc_f32_to_f16(_p(x), _p(out), _l(x.size))
    return out


def f16_bits_to_f32(h) -> np.ndarray:
    h = _c(h, np.uint16)
    out = np.empty(h.shape, np.float32)
    lib().orc_f16_to_f32(_p(h), _p(out), _l(h.size))
    return out


def f32_to_bf16_bits(x) -> np.ndarray:
    x = _c(x, np.float32)
    out = np.empty(x.shape, np.uint16)
    lib().orc_f32_to_bf16(_p(x), _p(out), _l(x.size))
    return out


def bf16_bits_to_f32(h) -> np.ndarray:
    h = _c(h, np.uint16)
    out = np.empty(h.shape, np.float32)
    lib().orc_bf16_to_f32(_p(h), _p(out), _l(h.size))
    return out


def to_act16(x, bf16: bool = False) -> np.ndarray:
    return f32_to_bf16_bits(x) if bf16 else f32_to_f16_bits(x)


def from_act16(h, bf16: bool = False) -> np.ndarray:
    return bf16_bits_to_f32(h) if bf16 else f16_bits_to_f32(h)


# --------------------------------------------------------------------------- generator
def fill_normal(n: int, seed: int, stream: int, first: int = 0, scale: float = 1.0) -> np.ndarray:
    """orc_fill_normal: counter-based ~N(0,1)*scale values (sum of eight uniform u16)."""
    out = np.empty(int(n), np.float32)
    lib().orc_fill_normal(_p(out), _l(n), C.c_uint64(seed), C.c_uint64(stream), C.c_uint64(first), C.c_float(scale))
    return out


def fill_uniform(n: int, seed: int, stream: int, first: int = 0) -> np.ndarray:
    out = np.empty(int(n), np.float32)
    lib().orc_fill_uniform(_p(out), _l(n), C.c_uint64(seed), C.c_uint64(stream), C.c_uint64(first))
    return out


# --------------------------------------------------------------------------- Q4 weights
def quantize_q4(W, awq_scales=None) -> np.ndarray:
    """orc_q4_from_f32: [N,K] f32 -> CPU blocks, uint8 [N, K/32, 20]."""
    W = _c(W, np.float32)
    N, K = W.shape
    assert K % 32 == 0
    blocks = np.empty((N, K // 32, 20), np.uint8)
    a = _c(awq_scales, np.float32) if awq_scales is not None else None
    lib().orc_q4_from_f32(_p(W), _l(N), _l(K), _p(a) if a is not None else None, _p(blocks))
    return blocks


def awq_inverse(awq_scales) -> np.ndarray:
    a = _c(awq_scales, np.float32)
    out = np.empty_like(a)
    lib().orc_awq_inverse(_p(a), _l(a.size), _p(out))
    return out


def extract_for_gpu(blocks):
    """orc_extract_for_gpu: CPU blocks -> (nibbles u8 [N,K/2], scales f32 [N,K/32])."""
    blocks = _c(blocks, np.uint8)
    N, nb, _ = blocks.shape
    nib = np.empty((N, nb * 16), np.uint8)
    sc = np.empty((N, nb), np.float32)
    lib().orc_extract_for_gpu(_p(blocks), _l(N), _l(nb * 32), _p(nib), _p(sc))
    return nib, sc


def q4_matvec(blocks, x, awq_inv=None, order: str = "scalar") -> np.ndarray:
    """orc_q4_matvec: the reference CPU GEMV; order 'scalar' or 'avx2'."""
    blocks = _c(blocks, np.uint8)
    N, nb, _ = blocks.shape
    x = _c(x, np.float32)
    assert x.size == nb * 32
    a = _c(awq_inv, np.float32) if awq_inv is not None else None
    y = np.empty(N, np.float32)
    lib().orc_q4_matvec(_p(blocks), _p(x), _l(N), _l(nb * 32), _p(a) if a is not None else None,
                        C.c_int(0 if order == "scalar" else 1), _p(y))
    return y


def q4_linear(blocks, X, awq_inv=None, order: str = "scalar") -> np.ndarray:
    X = _c(X, np.float32)
    return np.stack([q4_matvec(blocks, X[m], awq_inv, order) for m in range(X.shape[0])])


def q4_matvec_mt(blocks, x) -> np.ndarray:
    blocks = _c(blocks, np.uint8)
    N, nb, _ = blocks.shape
    x = _c(x, np.float32)
    y = np.empty(N, np.float32)
    lib().orc_q4_matvec_mt(_p(blocks), _p(x), _l(N), _l(nb * 32), _p(y))
    return y


def w4a16_matvec_f64(x, nibbles, scales, awq=None) -> np.ndarray:
    x = _c(x, np.float32)
    nibbles = _c(nibbles, np.uint8)
    scales = _c(scales, np.float32)
    N, nb = scales.shape
    a = _c(awq, np.float32) if awq is not None else None
    y = np.empty(N, np.float64)
    lib().orc_w4a16_matvec_f64(_p(x), _p(nibbles), _p(scales), _p(a) if a is not None else None, _l(N), _l(nb * 32),
                               _p(y))
    return y


def dequant_w4a16(nibbles, scales, awq=None, bf16: bool = False) -> np.ndarray:
    nibbles = _c(nibbles, np.uint8)
    scales = _c(scales, np.float32)
    N, nb = scales.shape
    a = _c(awq, np.float32) if awq is not None else None
    out = np.empty((N, nb * 32), np.uint16)
    lib().orc_dequant_w4a16(_p(nibbles), _p(scales), _p(a) if a is not None else None, _l(N), _l(nb * 32),
                            C.c_int(int(bf16)), _p(out))
    return out


# --------------------------------------------------------------------------- activations / W4A8
def quantize_q8(x16, bf16: bool = False):
    """orc_quantize_q8: 16-bit activations -> (int8 codes [K], f32 scales [K/32])."""
    x16 = _c(x16, np.uint16)
    K = x16.size
    assert K % 32 == 0
    xq = np.empty(K, np.int8)
    sc = np.empty(K // 32, np.float32)
    lib().orc_quantize_q8(_p(x16), _l(K), C.c_int(int(bf16)), _p(xq), _p(sc))
    return xq, sc


def quantize_q8_awq(x16, awq_inv, bf16: bool = False):
    """orc_quantize_q8_awq: int8 codes of x * awq_inv per group of 32."""
    x16 = _c(x16, np.uint16)
    awq_inv = _c(awq_inv, np.float32)
    K = x16.size
    assert K % 32 == 0 and awq_inv.size == K
    xq = np.empty(K, np.int8)
    sc = np.empty(K // 32, np.float32)
    lib().orc_quantize_q8_awq(_p(x16), _p(awq_inv), _l(K), C.c_int(int(bf16)), _p(xq), _p(sc))
    return xq, sc


def w4a8_idot(xq, nibbles) -> np.ndarray:
    xq = _c(xq, np.int8)
    nibbles = _c(nibbles, np.uint8)
    N = nibbles.shape[0]
    K = xq.size
    out = np.empty((N, K // 32), np.int32)
    lib().orc_w4a8_idot(_p(xq), _p(nibbles), _l(N), _l(K), _p(out))
    return out


def w4a8_matvec_f64(xq, xs, nibbles, wsc) -> np.ndarray:
    xq = _c(xq, np.int8)
    xs = _c(xs, np.float32)
    nibbles = _c(nibbles, np.uint8)
    wsc = _c(wsc, np.float32)
    N = nibbles.shape[0]
    y = np.empty(N, np.float64)
    lib().orc_w4a8_matvec_f64(_p(xq), _p(xs), _p(nibbles), _p(wsc), _l(N), _l(xq.size), _p(y))
    return y


def w4a8_matvec_reforder(xq, xs, nibbles, wsc) -> np.ndarray:
    xq = _c(xq, np.int8)
    xs = _c(xs, np.float32)
    nibbles = _c(nibbles, np.uint8)
    wsc = _c(wsc, np.float32)
    N = nibbles.shape[0]
    y = np.empty(N, np.float32)
    lib().orc_w4a8_matvec_reforder(_p(xq), _p(xs), _p(nibbles), _p(wsc), _l(N), _l(xq.size), _p(y))
    return y


def w4a8_matvec_b200(xq, xs, nibbles, wsc) -> np.ndarray:
    """orc_w4a8_matvec_b200: f32 result in the CUDA library's own summation order (bit-level check)."""
    xq = _c(xq, np.int8)
    xs = _c(xs, np.float32)
    nibbles = _c(nibbles, np.uint8)
    wsc = _c(wsc, np.float32)
    N = nibbles.shape[0]
    y = np.empty(N, np.float32)
    lib().orc_w4a8_matvec_b200(_p(xq), _p(xs), _p(nibbles), _p(wsc), _l(N), _l(xq.size), _p(y))
    return y


def x16_fixedpoint(x16, bf16: bool = False, awq=None):
    """orc_x16_fixedpoint: the library's 16-bit fixed-point activation codes (int32 [K]) and scales."""
    x16 = _c(x16, np.uint16)
    K = x16.size
    a = _c(awq, np.float32) if awq is not None else None
    v = np.empty(K, np.int32)
    sc = np.empty(K // 32, np.float32)
    lib().orc_x16_fixedpoint(_p(x16), _l(K), C.c_int(int(bf16)), _p(a) if a is not None else None, _p(v), _p(sc))
    return v, sc


def w4a16_matvec_b200(x16, nibbles, wsc, awq=None, bf16: bool = False) -> np.ndarray:
    """orc_w4a16_matvec_b200: f32 result exactly as the CUDA library computes it."""
    x16 = _c(x16, np.uint16)
    nibbles = _c(nibbles, np.uint8)
    wsc = _c(wsc, np.float32)
    a = _c(awq, np.float32) if awq is not None else None
    N = nibbles.shape[0]
    y = np.empty(N, np.float32)
    lib().orc_w4a16_matvec_b200(_p(x16), C.c_int(int(bf16)), _p(a) if a is not None else None, _p(nibbles), _p(wsc),
                                _l(N), _l(x16.size), _p(y))
    return y


def w4a8_matvec_mt(xq, xs, nibbles, wsc) -> np.ndarray:
    xq = _c(xq, np.int8)
    xs = _c(xs, np.float32)
    nibbles = _c(nibbles, np.uint8)
    wsc = _c(wsc, np.float32)
    N = nibbles.shape[0]
    y = np.empty(N, np.float32)
    lib().orc_w4a8_matvec_mt(_p(xq), _p(xs), _p(nibbles), _p(wsc), _l(N), _l(xq.size), _p(y))
    return y


# --------------------------------------------------------------------------- glue
def rms_norm_f64(x, w, eps: float) -> np.ndarray:
    x = _c(x, np.float32)
    w = _c(w, np.float32)
    out = np.empty_like(x)
    lib().orc_rms_norm_f64(_p(x), _p(w), _l(x.size), C.c_double(eps), _p(out))
    return out


def rms_norm_16(x16, w16, eps: float, bf16: bool = False) -> np.ndarray:
    x16 = _c(x16, np.uint16)
    w16 = _c(w16, np.uint16)
    out = np.empty_like(x16)
    lib().orc_rms_norm_16(_p(x16), _p(w16), _l(x16.size), C.c_float(eps), C.c_int(int(bf16)), _p(out))
    return out


def silu_mul_16(g16, u16, bf16: bool = False) -> np.ndarray:
    g16 = _c(g16, np.uint16)
    u16 = _c(u16, np.uint16)
    out = np.empty_like(g16)
    lib().orc_silu_mul_16(_p(g16), _p(u16), _l(g16.size), C.c_int(int(bf16)), _p(out))
    return out


def rope_tables_f32(head_dim: int, max_seq: int, theta: float):
    half = head_dim // 2
    cos = np.empty((max_seq, half), np.float32)
    sin = np.empty((max_seq, half), np.float32)
    lib().orc_rope_tables_f32(C.c_int(head_dim), C.c_int(max_seq), C.c_float(theta), _p(cos), _p(sin))
    return cos, sin


def rope_apply(v, n_heads: int, head_dim: int, cos_row, sin_row) -> np.ndarray:
    v = np.array(v, dtype=np.float32, copy=True).reshape(-1)
    cos_row = _c(cos_row, np.float32)
    sin_row = _c(sin_row, np.float32)
    lib().orc_rope_apply(_p(v), C.c_int(n_heads), C.c_int(head_dim), _p(cos_row), _p(sin_row))
    return v.reshape(n_heads, head_dim)


def attn_decode(q, kc, vc, seq_len: int, scale: float) -> np.ndarray:
    """orc_attn_decode: q [nh,hd], caches [nkv, stride, hd] (f32) -> [nh,hd]."""
    q = _c(q, np.float32)
    kc = _c(kc, np.float32)
    vc = _c(vc, np.float32)
    nh, hd = q.shape
    nkv, stride, _ = kc.shape
    out = np.empty((nh, hd), np.float32)
    lib().orc_attn_decode(_p(q), _p(kc), _p(vc), C.c_int(nh), C.c_int(nkv), C.c_int(seq_len), C.c_int(stride),
                          C.c_int(hd), C.c_float(scale), _p(out))
    return out


def attn_decode_f32(q, kc, vc, seq_len: int, scale: float) -> np.ndarray:
    """orc_attn_decode_f32: the reference's f32 loop order (timed baseline); same shapes as attn_decode."""
    q = _c(q, np.float32)
    kc = _c(kc, np.float32)
    vc = _c(vc, np.float32)
    nh, hd = q.shape
    nkv, stride, _ = kc.shape
    out = np.empty((nh, hd), np.float32)
    lib().orc_attn_decode_f32(_p(q), _p(kc), _p(vc), C.c_int(nh), C.c_int(nkv), C.c_int(seq_len), C.c_int(stride),
                              C.c_int(hd), C.c_float(scale), _p(out))
    return out


# --------------------------------------------------------------------------- routing
def normalize_importance(scores) -> np.ndarray:
    s = _c(scores, np.float64)
    out = np.empty_like(s)
    lib().orc_normalize_importance(_p(s), C.c_int(s.size), _p(out))
    return out


def use_w4a8(importance: float, threshold: float = 0.7, no_w4a8: bool = False) -> bool:
    return bool(lib().orc_use_w4a8(float(importance), float(threshold), int(no_w4a8)))


def set_threads(n: int) -> None:
    lib().orc_set_threads(C.c_int(int(n)))


def have_avx2() -> bool:
    return bool(lib().orc_have_avx2())
