"""Independent numpy restatement of the oracle -- TEST INFRASTRUCTURE ONLY.

Written separately from ``nve_oracle.c`` (vectorised numpy instead of scalar C loops) so that
the two can be checked against each other; a disagreement means one of them misreads the
reference.  Citations are reference-project paths.
"""
from __future__ import annotations

import numpy as np

_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)
_GOLDEN = np.uint64(0x9E3779B97F4A7C15)
_STREAM = np.uint64(0xD6E8FEB86659FD93)
_IH8 = np.float32(float.fromhex("0x1.3988e2p-16"))


def _mix64(z: np.ndarray) -> np.ndarray:
    z = np.asarray(z, dtype=np.uint64)
    with np.errstate(over="ignore"):
        z = (z ^ (z >> np.uint64(30))) * _M1
        z = (z ^ (z >> np.uint64(27))) * _M2
    return z ^ (z >> np.uint64(31))


def _state(seed: int, stream: int) -> np.uint64:
    with np.errstate(over="ignore"):
        return _mix64(np.uint64(seed) ^ (np.uint64(stream) * _STREAM))


def fill_normal(n: int, seed: int, stream: int, first: int = 0, scale: float = 1.0) -> np.ndarray:
    """Counter-based generator: sum of eight uniform 16-bit fields, centred and scaled."""
    st = _state(seed, stream)
    i = np.arange(first, first + n, dtype=np.uint64)
    with np.errstate(over="ignore"):
        a = _mix64(st + (np.uint64(2) * i + np.uint64(1)) * _GOLDEN)
        b = _mix64(st + (np.uint64(2) * i + np.uint64(2)) * _GOLDEN)
    s = np.zeros(n, dtype=np.int64)
    for j in range(4):
        s += ((a >> np.uint64(16 * j)) & np.uint64(0xFFFF)).astype(np.int64)
        s += ((b >> np.uint64(16 * j)) & np.uint64(0xFFFF)).astype(np.int64)
    z = (s - 262140).astype(np.float32) * _IH8
    return (z * np.float32(scale)).astype(np.float32)


def fill_uniform(n: int, seed: int, stream: int, first: int = 0) -> np.ndarray:
    st = _state(seed, stream)
    i = np.arange(first, first + n, dtype=np.uint64)
    with np.errstate(over="ignore"):
        a = _mix64(st + (np.uint64(2) * i + np.uint64(1)) * _GOLDEN)
    return (a >> np.uint64(40)).astype(np.float32) * np.float32(2.0**-24)


def _round_half_away(v: np.ndarray) -> np.ndarray:
    return np.sign(v) * np.floor(np.abs(v) + np.float32(0.5))


def quantize_q4(W: np.ndarray):
    """src/quantize.rs:711-731 over a whole matrix: returns (q in [0,15] as [N,K] u8, scales [N,K/32] f32)."""
    W = np.asarray(W, np.float32)
    N, K = W.shape
    B = W.reshape(N, K // 32, 32)
    amax = np.abs(B).max(axis=2)
    scale = np.where(amax > 0, amax / np.float32(7.0), np.float32(0.0)).astype(np.float32)
    with np.errstate(divide="ignore"):
        inv = np.where(scale > 0, np.float32(1.0) / scale, np.float32(0.0)).astype(np.float32)
    t = (B * inv[:, :, None]).astype(np.float32)
    # |t| <= 7 + rounding, so floor(|t| + 0.5) is exact in f32
    q = np.clip(_round_half_away(t), -8, 7).astype(np.int32) + 8
    return q.reshape(N, K).astype(np.uint8), scale


def pack_cpu(q: np.ndarray, scales: np.ndarray) -> np.ndarray:
    """CPU block bytes [N, K/32, 20]: f32 LE scale then byte i = q[2i] | q[2i+1] << 4 (src/quantize.rs:720-730)."""
    N, K = q.shape
    qb = q.reshape(N, K // 32, 16, 2)
    by = (qb[..., 0] | (qb[..., 1] << 4)).astype(np.uint8)
    out = np.empty((N, K // 32, 20), np.uint8)
    out[:, :, :4] = scales.astype("<f4").view(np.uint8).reshape(N, K // 32, 4)
    out[:, :, 4:] = by
    return out


def pack_gpu(q: np.ndarray) -> np.ndarray:
    """Device nibbles [N, K/2]: byte j of a block = q[j] | q[j+16] << 4 (src/quantize.rs:450-458)."""
    N, K = q.shape
    qb = q.reshape(N, K // 32, 2, 16)
    return (qb[:, :, 0, :] | (qb[:, :, 1, :] << 4)).astype(np.uint8).reshape(N, K // 2)


def unpack_gpu(nibbles: np.ndarray) -> np.ndarray:
    """Inverse of pack_gpu: signed values q-8 as int32 [N,K]."""
    N, half = nibbles.shape
    nb = nibbles.reshape(N, half // 16, 16).astype(np.int32)
    lo = (nb & 0xF) - 8
    hi = (nb >> 4) - 8
    return np.concatenate([lo, hi], axis=2).reshape(N, half * 2)


def w4a16_matvec(x: np.ndarray, nibbles: np.ndarray, scales: np.ndarray, awq=None) -> np.ndarray:
    """y[n] = sum_b scale[n,b] * sum_e (q-8) * x  in f64 (src/quantize.rs:853-879 with an exact sum)."""
    x = np.asarray(x, np.float32)
    if awq is not None:
        x = (x * np.asarray(awq, np.float32)).astype(np.float32)
    q = unpack_gpu(nibbles).astype(np.float64)
    N, K = q.shape
    bs = (q * x.astype(np.float64)[None, :]).reshape(N, K // 32, 32).sum(axis=2)
    return (bs * scales.astype(np.float64)).sum(axis=1)


def quantize_q8(x16_as_f32: np.ndarray):
    """cuda/nve_kernels.cu:712-745 on already-rounded activations given as f32."""
    x = np.asarray(x16_as_f32, np.float32).reshape(-1, 32)
    amax = np.abs(x).max(axis=1)
    scale = np.where(amax > 0, amax / np.float32(127.0), np.float32(1.0)).astype(np.float32)
    inv = (np.float32(1.0) / scale).astype(np.float32)
    t = (x * inv[:, None]).astype(np.float32)
    q = np.clip(np.rint(t), -127, 127).astype(np.int8)  # rint: half to even
    return q.reshape(-1), scale


def w4a8_idot(xq: np.ndarray, nibbles: np.ndarray) -> np.ndarray:
    q = unpack_gpu(nibbles).astype(np.int64)
    N, K = q.shape
    return (q * xq.astype(np.int64)[None, :]).reshape(N, K // 32, 32).sum(axis=2).astype(np.int32)


def w4a8_matvec(xq, xs, nibbles, wsc) -> np.ndarray:
    I = w4a8_idot(xq, nibbles).astype(np.float64)
    return (I * wsc.astype(np.float64) * xs.astype(np.float64)[None, :]).sum(axis=1)


def rms_norm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    """src/ops.rs:12-30."""
    x64 = np.asarray(x, np.float64)
    inv = 1.0 / np.sqrt((x64 * x64).sum() / x64.size + eps)
    return (x64 * inv * np.asarray(w, np.float64)).astype(np.float32)
