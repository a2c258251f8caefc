"""Small helpers shared by the GPU parity tests."""
import numpy as np
import torch


def dev(a: np.ndarray, dtype=None) -> torch.Tensor:
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.view(dtype)


def f16_bits(t: torch.Tensor) -> np.ndarray:
    return t.detach().contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def rel_rms_err(y, ref) -> float:
    """max |y - ref| / RMS(ref): the tolerance form stated for W4A16 and scaled outputs."""
    y = np.asarray(y, np.float64).reshape(-1)
    ref = np.asarray(ref, np.float64).reshape(-1)
    rms = np.sqrt(np.mean(ref * ref))
    return float(np.max(np.abs(y - ref)) / max(rms, 1e-30))


TOL = 1e-2  # max-abs <= 1e-2 * RMS(reference output), fp32 accumulation


def same_f16(a_bits: np.ndarray, b_bits: np.ndarray, bf16: bool = False) -> bool:
    """Bit equality of two 16-bit float arrays, except that any NaN equals any NaN (host and device
    conversions pick different NaN payloads)."""
    a = np.asarray(a_bits, np.uint16).reshape(-1)
    b = np.asarray(b_bits, np.uint16).reshape(-1)
    if a.shape != b.shape:
        return False
    if bf16:
        nan_a = ((a & 0x7F80) == 0x7F80) & ((a & 0x007F) != 0)
        nan_b = ((b & 0x7F80) == 0x7F80) & ((b & 0x007F) != 0)
    else:
        nan_a = ((a & 0x7C00) == 0x7C00) & ((a & 0x03FF) != 0)
        nan_b = ((b & 0x7C00) == 0x7C00) & ((b & 0x03FF) != 0)
    return bool(np.all((a == b) | (nan_a & nan_b)))
