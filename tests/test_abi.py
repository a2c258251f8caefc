"""CPU: the shared library loads and exports every symbol include/nve_kernels.h declares, the ctypes
binding covers exactly those symbols, and launchers reject bad arguments without touching a device."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
HEADER = os.path.join(ROOT, "include", "nve_kernels.h")

# The 27 symbols the reference exports from cuda/nve_kernels.cu (26 bound in src/cuda_kernels.rs:57-289
# plus nve_run_microbench, called from cuda/bench_main.cu).
REFERENCE_EXPORTS = """
nve_rms_norm_f16 nve_layer_norm_f16 nve_rope_f16_decode nve_rope_f16_prefill nve_rope_f16_decode_dyn
nve_matvec_f16 nve_matvec_w4a16 nve_dequant_w4a16 nve_qkv_matvec_w4a16 nve_quantize_f16_q8 nve_matvec_w4a8
nve_flash_decode_f16 nve_flash_decode_dyn nve_kv_cache_write_f16 nve_add_inplace_f16 nve_silu_mul_f16
nve_d2d_copy nve_graph_init nve_graph_begin_capture nve_graph_end_capture nve_graph_launch nve_graph_ready
nve_graph_destroy nve_graph_d_pos nve_graph_d_seqlen nve_graph_capture_stream nve_run_microbench
""".split()


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return re.findall(r"NVE_API\s+[\w\s\*]+?\b(nve_\w+)\s*\(", text)


@pytest.fixture(scope="module")
def lib():
    from nve_b200 import build, _ffi

    build.build()  # nvcc cross-compiles for sm_100a without a GPU
    return _ffi.load()


def test_header_declares_reference_abi():
    names = declared_symbols()
    assert len(names) == len(set(names))
    missing = [n for n in REFERENCE_EXPORTS if n not in names]
    assert not missing, missing
    assert len(REFERENCE_EXPORTS) == 27


def test_library_exports_every_declared_symbol(lib):
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} is declared in include/nve_kernels.h but not exported"


def test_binding_matches_header(lib):
    from nve_b200 import _ffi

    assert sorted(_ffi.SIGNATURES) == sorted(declared_symbols())


def test_argument_counts_match_header():
    from nve_b200 import _ffi

    text = re.sub(r"/\*.*?\*/", "", open(HEADER).read(), flags=re.S)
    for name, (_, args) in _ffi.SIGNATURES.items():
        m = re.search(r"\b" + name + r"\s*\(([^;]*?)\)\s*;", text, flags=re.S)
        assert m, name
        params = m.group(1).strip()
        n = 0 if params in ("", "void") else params.count(",") + 1
        assert n == len(args), (name, n, len(args))


def test_host_side_argument_validation(lib):
    """Launchers validate before launching: these calls never reach a device."""
    from nve_b200 import _ffi

    assert lib.nve_b200_version().startswith(b"nve-b200")
    m = _ffi.W4Matrix(0x1000, 0x1000, 0x1000, None, 8)
    assert lib.nve_b200_matvec_w4a8_multi(0x1000, 0x1000, C.byref(m), 1, 48, 0, None) == 1  # K % 32 != 0
    assert lib.nve_b200_matvec_w4a8_multi(None, 0x1000, C.byref(m), 1, 64, 0, None) == 2  # NULL activations
    assert lib.nve_b200_matvec_w4a8_multi(0x1000, 0x1000, C.byref(m), 4, 64, 0, None) == 1  # too many matrices
    assert lib.nve_b200_matvec_w4a16_multi(0x1000, 7, None, C.byref(m), 1, 64, 0, None) == 4  # bad dtype
    assert lib.nve_b200_quantize_q8(0x1000, 0x1000, 0x1000, 33, 0, None) == 1
    assert lib.nve_b200_quantize_q8(0x1000, None, 0x1000, 32, 0, None) == 2
    assert lib.nve_b200_q4_quantize(0x1008, None, 0x1000, 0x1000, 4, 64, None) == 3  # misaligned weights
    assert lib.nve_b200_last_status() == 3
    # reference-signature launchers record the reason instead of returning it
    lib.nve_quantize_f16_q8(None, None, None, 64, None)
    assert lib.nve_b200_last_status() == 2
    lib.nve_flash_decode_f16(0x1000, 0x1000, 0x1000, 0x1000, 32, 8, 16, 80, 0.1, None)  # head_dim % 32 != 0
    assert lib.nve_b200_last_status() == 1
    assert lib.nve_graph_ready() == 0
    lib.nve_graph_launch(0, 1, None)  # not captured: skipped, as the reference does
    assert lib.nve_b200_last_status() != 0


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from nve_b200 import _ffi

    monkeypatch.setattr(_ffi, "_lib", None)
    monkeypatch.setattr(_ffi, "LIB_PATH", str(tmp_path / "libnve_kernels.so"))
    with pytest.raises(ImportError):
        _ffi.load()
