"""GPU: the oracle pinned against the reference project's own CUDA kernels.

oracle/_ref/libnve_kernels_ref.so is the reference's cuda/nve_kernels.cu compiled unmodified for sm_100a by
oracle/Makefile (IEEE arithmetic; a second build uses the reference's own --use_fast_math flag).  The
reference has no CPU implementation and no test for the activation quantizer or the W4A8 GEMV, so running
its kernels on the same seeded inputs is what ties the oracle restatement -- and through it this library --
to the reference's behaviour.
"""
import ctypes as C
import os

import numpy as np
import pytest

from helpers import TOL, dev, f16_bits, rel_rms_err

pytestmark = pytest.mark.gpu

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
REF = os.path.join(ROOT, "oracle", "_ref", "libnve_kernels_ref.so")
REF_FAST = os.path.join(ROOT, "oracle", "_ref", "libnve_kernels_ref_fastmath.so")


def _load(path):
    if not os.path.exists(path):
        pytest.skip(f"{os.path.relpath(path, ROOT)} not built (needs the reference checkout: make -C oracle ref)")
    lib = C.CDLL(path)
    P, I = C.c_void_p, C.c_int
    lib.nve_quantize_f16_q8.argtypes = [P, P, P, I, P]
    lib.nve_matvec_w4a8.argtypes = [P, P, P, P, P, I, I, P]
    lib.nve_matvec_w4a16.argtypes = [P, P, P, P, P, I, I, P]
    lib.nve_rms_norm_f16.argtypes = [P, P, P, I, C.c_float, P]
    for f in (lib.nve_quantize_f16_q8, lib.nve_matvec_w4a8, lib.nve_matvec_w4a16, lib.nve_rms_norm_f16):
        f.restype = None
    return lib


def _case(orc, N, K, seed):
    W = orc.fill_normal(N * K, seed, 1, scale=0.02).reshape(N, K)
    blocks = orc.quantize_q4(W)
    nib, sc = orc.extract_for_gpu(blocks)
    x16 = orc.to_act16(orc.fill_normal(K, seed, 2))
    return blocks, nib, sc, x16


@pytest.mark.parametrize("K", [2048, 4096, 8192])
def test_reference_quantizer_matches_oracle_and_library(cuda, orc, K):
    from nve_b200 import cuda_kernels as ck

    torch = cuda
    ref = _load(REF)
    x16 = orc.to_act16(orc.fill_normal(K, 901, K) * 2.5)
    dx = dev(x16, torch.float16)
    xq = torch.empty(K, dtype=torch.int8, device="cuda")
    xs = torch.empty(K // 32, dtype=torch.float32, device="cuda")
    ref.nve_quantize_f16_q8(dx.data_ptr(), xq.data_ptr(), xs.data_ptr(), K, None)
    torch.cuda.synchronize()
    eq, es = orc.quantize_q8(x16)
    assert np.array_equal(xq.cpu().numpy(), eq)
    assert np.array_equal(xs.cpu().numpy().view(np.uint32), es.view(np.uint32))
    mq, ms = ck.quantize_f16_q8(dx)
    assert torch.equal(mq, xq) and torch.equal(ms, xs)


@pytest.mark.parametrize("N,K", [(2048, 2048), (512, 2048), (8192, 2048), (2048, 8192), (1024, 4096)])
def test_reference_w4a8_matches_oracle_and_library(cuda, orc, N, K):
    from nve_b200 import cuda_kernels as ck

    torch = cuda
    ref = _load(REF)
    _, nib, sc, x16 = _case(orc, N, K, 910 + N % 97)
    xq, xs = orc.quantize_q8(x16)
    dxq, dxs, dn, ds = dev(xq), dev(xs), dev(nib), dev(sc)
    out = torch.empty(N, dtype=torch.float16, device="cuda")
    ref.nve_matvec_w4a8(dxq.data_ptr(), dxs.data_ptr(), dn.data_ptr(), ds.data_ptr(), out.data_ptr(), N, K, None)
    torch.cuda.synchronize()
    got = out.float().cpu().numpy()
    exact = orc.w4a8_matvec_f64(xq, xs, nib, sc)
    assert rel_rms_err(got, exact) < 5e-3  # one f16 rounding of the output
    # the oracle's restatement of the reference kernel's own summation order reproduces it (up to the rare
    # double rounding of f32 -> f16)
    reforder = orc.f32_to_f16_bits(orc.w4a8_matvec_reforder(xq, xs, nib, sc))
    assert np.mean(f16_bits(out) == reforder) > 0.999
    mine = ck.matvec_w4a8(dxq, dxs, dn, ds, N, K).float().cpu().numpy().reshape(-1)
    assert rel_rms_err(mine, got) < 5e-3


@pytest.mark.parametrize("N,K", [(8192, 2048), (2048, 8192)])
def test_reference_w4a16_matches_cpu_oracle_and_library(cuda, orc, N, K):
    from nve_b200 import cuda_kernels as ck

    torch = cuda
    ref = _load(REF)
    blocks, nib, sc, x16 = _case(orc, N, K, 920 + N % 97)
    dx, dn, ds = dev(x16, torch.float16), dev(nib), dev(sc)
    out = torch.empty(N, dtype=torch.float16, device="cuda")
    ref.nve_matvec_w4a16(dx.data_ptr(), dn.data_ptr(), ds.data_ptr(), None, out.data_ptr(), N, K, None)
    torch.cuda.synchronize()
    cpu = orc.q4_matvec(blocks, orc.from_act16(x16), order="scalar")
    assert rel_rms_err(out.float().cpu().numpy(), cpu) < 5e-3
    mine = ck.fused_matvec_w4a16(dx, dn, ds, None, N, K).float().cpu().numpy().reshape(-1)
    assert rel_rms_err(mine, out.float().cpu().numpy()) < 5e-3
    assert rel_rms_err(mine, cpu) < TOL


def test_reference_fastmath_build_differs_only_in_rounding(cuda, orc):
    """The reference ships with --use_fast_math (build.rs:66-75): approximate division may move a scale by an
    ulp and a code by one step.  The IEEE restatement is the defined behaviour; this bounds the difference."""
    torch = cuda
    fast = _load(REF_FAST)
    K = 8192
    x16 = orc.to_act16(orc.fill_normal(K, 930, 1) * 2.5)
    dx = dev(x16, torch.float16)
    xq = torch.empty(K, dtype=torch.int8, device="cuda")
    xs = torch.empty(K // 32, dtype=torch.float32, device="cuda")
    fast.nve_quantize_f16_q8(dx.data_ptr(), xq.data_ptr(), xs.data_ptr(), K, None)
    torch.cuda.synchronize()
    eq, es = orc.quantize_q8(x16)
    d = np.abs(xq.cpu().numpy().astype(np.int32) - eq.astype(np.int32))
    assert d.max() <= 1 and np.mean(d != 0) < 0.01
    assert np.max(np.abs(xs.cpu().numpy() - es) / es) < 1e-6


def test_reference_rms_norm_within_rounding(cuda, orc):
    from nve_b200 import cuda_kernels as ck

    torch = cuda
    ref = _load(REF)
    n = 4096
    x16 = orc.to_act16(orc.fill_normal(n, 940, 1))
    w16 = orc.to_act16(1.0 + 0.1 * orc.fill_normal(n, 940, 2))
    dx, dw = dev(x16, torch.float16), dev(w16, torch.float16)
    out = torch.empty(n, dtype=torch.float16, device="cuda")
    ref.nve_rms_norm_f16(dx.data_ptr(), dw.data_ptr(), out.data_ptr(), n, 1e-5, None)
    torch.cuda.synchronize()
    mine = ck.fused_rms_norm(dx, dw, 1e-5)
    diff = np.abs(out.float().cpu().numpy() - mine.float().cpu().numpy())
    assert np.all(diff <= np.abs(mine.float().cpu().numpy()) * 2.0**-10 + 1e-7)  # at most one f16 ulp apart
