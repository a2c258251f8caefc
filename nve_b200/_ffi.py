"""ctypes binding of libnve_kernels.so (the C ABI declared in include/nve_kernels.h).

This is the Python analogue of the ``extern "C"`` block in the reference's src/cuda_kernels.rs:57-289:
plain pointers and sizes, nothing else.  The library is loaded from ``nve_b200/lib``; if it is missing
the import of any kernel wrapper fails loudly -- there is no CPU or PyTorch fallback.
"""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "lib", "libnve_kernels.so")

NVE_DT_F16, NVE_DT_BF16, NVE_DT_F32 = 0, 1, 2

STATUS_NAMES = {
    0: "NVE_OK",
    1: "NVE_ERR_BAD_SHAPE",
    2: "NVE_ERR_BAD_POINTER",
    3: "NVE_ERR_BAD_ALIGNMENT",
    4: "NVE_ERR_BAD_DTYPE",
    5: "NVE_ERR_TOO_LARGE",
    6: "NVE_ERR_CUDA",
    7: "NVE_ERR_TIMEOUT",
}


class NveKernelError(RuntimeError):
    """A launcher of libnve_kernels.so reported a non-zero status."""

    def __init__(self, fn: str, status: int, cuda_error: int = 0):
        self.fn, self.status, self.cuda_error = fn, status, cuda_error
        msg = f"{fn}: {STATUS_NAMES.get(status, status)}"
        if status == 6:
            msg += f" (cudaError {cuda_error})"
        super().__init__(msg)


class W4Matrix(C.Structure):
    """nve_b200_w4_matrix."""

    _fields_ = [
        ("nibbles", C.c_void_p),
        ("scales", C.c_void_p),
        ("out", C.c_void_p),
        ("residual", C.c_void_p),
        ("N", C.c_int),
    ]


class DecodeLayer(C.Structure):
    """nve_b200_decode_layer."""

    _fields_ = [
        ("nibbles", C.c_void_p * 7),
        ("scales", C.c_void_p * 7),
        ("awq", C.c_void_p * 4),
        ("input_norm", C.c_void_p),
        ("post_attn_norm", C.c_void_p),
        ("k_cache", C.c_void_p),
        ("v_cache", C.c_void_p),
        ("use_w4a8", C.c_int),
        ("reserved", C.c_int),
    ]


class DecodeModel(C.Structure):
    """nve_b200_decode_model."""

    _fields_ = [
        ("hidden", C.c_int), ("ffn", C.c_int), ("num_heads", C.c_int), ("num_kv_heads", C.c_int),
        ("head_dim", C.c_int), ("max_seq", C.c_int), ("num_layers", C.c_int),
        ("norm_eps", C.c_float), ("attn_scale", C.c_float),
        ("rope_cos", C.c_void_p), ("rope_sin", C.c_void_p),
        ("final_norm", C.c_void_p), ("lm_nibbles", C.c_void_p), ("lm_scales", C.c_void_p), ("logits", C.c_void_p),
        ("vocab", C.c_int), ("lm_use_w4a8", C.c_int),
    ]


_P, _I, _F, _S = C.c_void_p, C.c_int, C.c_float, C.c_size_t
_LL, _ULL = C.c_longlong, C.c_ulonglong

# name -> (restype, argtypes).  Order and types follow include/nve_kernels.h exactly.
SIGNATURES = {
    # ---- reference ABI
    "nve_rms_norm_f16": (None, [_P, _P, _P, _I, _F, _P]),
    "nve_layer_norm_f16": (None, [_P, _P, _P, _P, _I, _F, _P]),
    "nve_rope_f16_decode": (None, [_P, _P, _P, _P, _I, _I, _I, _P]),
    "nve_rope_f16_prefill": (None, [_P, _P, _P, _P, _I, _I, _I, _I, _I, _P]),
    "nve_rope_f16_decode_dyn": (None, [_P, _P, _P, _P, _I, _I, _I, _P, _P]),
    "nve_matvec_f16": (None, [_P, _P, _P, _I, _I, _P]),
    "nve_matvec_w4a16": (None, [_P, _P, _P, _P, _P, _I, _I, _P]),
    "nve_dequant_w4a16": (None, [_P, _P, _P, _P, _I, _I, _P]),
    "nve_qkv_matvec_w4a16": (None, [_P, _P, _P, _P, _I, _P, _P, _P, _I, _P, _P, _P, _I, _P, _P, _P, _I, _P]),
    "nve_quantize_f16_q8": (None, [_P, _P, _P, _I, _P]),
    "nve_matvec_w4a8": (None, [_P, _P, _P, _P, _P, _I, _I, _P]),
    "nve_flash_decode_f16": (None, [_P, _P, _P, _P, _I, _I, _I, _I, _F, _P]),
    "nve_flash_decode_dyn": (None, [_P, _P, _P, _P, _I, _I, _P, _I, _F, _I, _P]),
    "nve_kv_cache_write_f16": (None, [_P, _P, _P, _P, _P, _I, _I, _I, _P]),
    "nve_add_inplace_f16": (None, [_P, _P, _I, _P]),
    "nve_silu_mul_f16": (None, [_P, _P, _I, _P]),
    "nve_d2d_copy": (None, [_P, _P, _S, _P]),
    "nve_graph_init": (None, []),
    "nve_graph_begin_capture": (None, []),
    "nve_graph_end_capture": (None, []),
    "nve_graph_launch": (None, [_I, _I, _P]),
    "nve_graph_ready": (_I, []),
    "nve_graph_destroy": (None, []),
    "nve_graph_d_pos": (_P, []),
    "nve_graph_d_seqlen": (_P, []),
    "nve_graph_capture_stream": (_P, []),
    "nve_run_microbench": (None, [_I, _I, _I, _I, _I, _I]),
    # ---- additive
    "nve_b200_last_status": (_I, []),
    "nve_b200_last_cuda_error": (_I, []),
    "nve_b200_version": (C.c_char_p, []),
    "nve_b200_launch_count": (_ULL, []),
    "nve_b200_set_pdl": (_I, [_I]),
    "nve_b200_set_attn_decode_kernel": (_I, [_I]),
    "nve_b200_quantize_q8": (_I, [_P, _P, _P, _I, _I, _P]),
    "nve_b200_quantize_q8_awq": (_I, [_P, _P, _P, _P, _I, _I, _P]),
    "nve_b200_rmsnorm_quantize_q8": (_I, [_P, _P, _P, _P, _P, _I, _F, _I, _P]),
    "nve_b200_rms_norm": (_I, [_P, _P, _P, _I, _F, _I, _P]),
    "nve_b200_silu_mul_quantize_q8": (_I, [_P, _P, _P, _P, _P, _I, _I, _P]),
    "nve_b200_silu_mul_x16": (_I, [_P, _P, _P, _P, _P, _P, _P, _I, _I, _P]),
    "nve_b200_silu_mul": (_I, [_P, _P, _I, _I, _P]),
    "nve_b200_add_inplace": (_I, [_P, _P, _I, _I, _P]),
    "nve_b200_matvec_w4a8_multi": (_I, [_P, _P, C.POINTER(W4Matrix), _I, _I, _I, _P]),
    "nve_b200_matvec_w4a16_multi": (_I, [_P, _I, _P, C.POINTER(W4Matrix), _I, _I, _I, _P]),
    "nve_b200_matvec_w4a16_planes_multi": (_I, [_P, _P, _P, C.POINTER(W4Matrix), _I, _I, _I, _P]),
    "nve_b200_rmsnorm_matvec_w4a8_multi": (_I, [_P, _P, _F, _I, C.POINTER(W4Matrix), _I, _I, _I, _P]),
    "nve_b200_rmsnorm_matvec_w4a8_awq_multi": (_I, [_P, _P, _F, _I, _P, C.POINTER(W4Matrix), _I, _I, _I, _P]),
    "nve_b200_rmsnorm_matvec_w4a16_multi": (_I, [_P, _P, _F, _I, _P, C.POINTER(W4Matrix), _I, _I, _I, _P]),
    "nve_b200_rmsnorm_gateup_silu_w4a8": (_I, [_P, _P, _F, _I, _P, C.POINTER(W4Matrix), C.POINTER(W4Matrix), _P, _I, _P]),
    "nve_b200_rmsnorm_gateup_silu_w4a16": (_I, [_P, _P, _F, _I, _P, C.POINTER(W4Matrix), C.POINTER(W4Matrix), _P, _I, _P]),
    "nve_b200_rms_norm_rows": (_I, [_P, _P, _P, _I, _I, _F, _I, _P]),
    "nve_b200_add_rms_norm_rows": (_I, [_P, _P, _P, _P, _I, _I, _F, _I, _P]),
    "nve_b200_kv_cache_write_rows": (_I, [_P, _P, _P, _P, _I, _I, _I, _I, _I, _P]),
    "nve_b200_attn_prefill_causal": (_I, [_P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _P]),
    "nve_b200_rmsnorm_gateup_silu_q8_w4a8": (_I, [_P, _P, _F, _I, _P, C.POINTER(W4Matrix), C.POINTER(W4Matrix), _P, _I, _P, _P, _P, _P]),
    "nve_b200_rmsnorm_gateup_silu_x16_w4a16": (_I, [_P, _P, _F, _I, _P, C.POINTER(W4Matrix), C.POINTER(W4Matrix), _P, _I, _P, _P, _P,
                                                    _P, _P, _P]),
    "nve_b200_quantize_matvec_w4a8_multi": (_I, [_P, _I, _P, C.POINTER(W4Matrix), _I, _I, _P]),
    "nve_b200_quantize_matvec_w4a8_allreduce": (_I, [_P, _I, _P, C.POINTER(W4Matrix), _I, _P]),
    "nve_b200_attn_decode_fused": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _F, _P]),
    "nve_b200_attn_decode_fused_batch": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _F, _P]),
    "nve_b200_w4a8_idot": (_I, [_P, _P, _P, _I, _I, _P]),
    "nve_b200_dequant_w4a16": (_I, [_P, _P, _P, _P, _I, _I, _I, _P]),
    "nve_b200_q4_quantize": (_I, [_P, _P, _P, _P, _I, _I, _P]),
    "nve_b200_q4_repack_blocks": (_I, [_P, _P, _P, _I, _I, _P]),
    "nve_b200_gemm_w4a16_scratch_bytes": (_S, [_I, _I, _I]),
    "nve_b200_gemm_w4a16": (_I, [_P, _I, _P, _P, _P, _I, _I, _I, _I, _P, _S, _P]),
    "nve_b200_gemm_w4a16_multi_scratch_bytes": (_S, [_I, _P, _I, _I]),
    "nve_b200_gemm_w4a16_multi": (_I, [_P, _I, C.POINTER(W4Matrix), _I, _I, _I, _I, _P, _S, _P]),
    "nve_b200_gemm_error": (_I, [_I]),
    "nve_b200_gemm_w4a16_noalloc": (_I, [_P, _I, _P, _P, _P, _I, _I, _I, _I, _P]),
    "nve_b200_decode_step_workspace_bytes": (_S, [C.POINTER(DecodeModel)]),
    "nve_b200_decode_step_init": (_I, [_P, _S, _P]),
    "nve_b200_decode_step": (_I, [C.POINTER(DecodeModel), _P, _P, _P, _P, _P, _S, _P]),
    "nve_b200_decode_step_error": (_I, [_P, _I]),
    "nve_b200_decode_step_set_prefetch": (_I, [_I]),
    "nve_b200_decode_step_wait_probe": (_I, [_P, _ULL, _P]),
    "nve_b200_decode_step_set_trace": (None, [_P]),
    "nve_b200_tp_create": (_I, [_I, _I, _I, _P]),
    "nve_b200_tp_connect": (_I, [_P]),
    "nve_b200_tp_world": (_I, []),
    "nve_b200_tp_error": (_I, [_I]),
    "nve_b200_tp_destroy": (_I, []),
    "nve_b200_matvec_w4a8_allreduce": (_I, [_P, _P, C.POINTER(W4Matrix), _I, _I, _P]),
    "nve_b200_matvec_w4a16_allreduce": (_I, [_P, _I, _P, C.POINTER(W4Matrix), _I, _I, _P]),
    "nve_b200_matvec_w4a16_planes_allreduce": (_I, [_P, _P, _P, C.POINTER(W4Matrix), _I, _I, _P]),
    "nve_b200_fill_normal": (_I, [_P, _LL, _ULL, _ULL, _ULL, _F, _P]),
    "nve_b200_fill_normal_16": (_I, [_P, _LL, _ULL, _ULL, _ULL, _F, _I, _P]),
}

_lib = None


def load() -> C.CDLL:
    """Load the library and bind every declared symbol; raises if the library or a symbol is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m nve_b200.build` (nvcc, sm_100a). "
            "There is no fallback path."
        )
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(fn: str, status: int) -> None:
    """Raise NveKernelError for a non-zero status returned by an nve_b200_* launcher."""
    if status != 0:
        raise NveKernelError(fn, status, load().nve_b200_last_cuda_error())


def check_last(fn: str) -> None:
    """Raise if the most recent reference-signature (void) launcher recorded an error."""
    lib = load()
    st = lib.nve_b200_last_status()
    if st != 0:
        raise NveKernelError(fn, st, lib.nve_b200_last_cuda_error())
