"""GPU parity: the batched W4A16 GEMM (mma.sync kernel up to 8 batch rows, tcgen05 kernel above) against the
reference's CPU semantics (q4_linear: one f32 GEMV per row of X, src/quantize.rs:1057-1075) on the same
16-bit-rounded activations."""
import os
import subprocess
import sys

import numpy as np
import pytest

from helpers import TOL, dev, rel_rms_err
from oracle import np_oracle as npo

pytestmark = pytest.mark.gpu


def _case(orc, M, N, K, seed, bf):
    W = orc.fill_normal(N * K, seed, 1, scale=0.02).reshape(N, K)
    nib, sc = orc.extract_for_gpu(orc.quantize_q4(W))
    X16 = orc.to_act16(orc.fill_normal(M * K, seed, 2), bf).reshape(M, K)
    Wq = npo.unpack_gpu(nib).astype(np.float64) * np.repeat(sc.astype(np.float64), 32, axis=1)
    ref = orc.from_act16(X16, bf).astype(np.float64) @ Wq.T
    return nib, sc, X16, ref


@pytest.mark.parametrize("M,N,K", [(16, 128, 64), (16, 128, 512), (1, 256, 1024), (8, 384, 2048), (32, 1024, 4096),
                                    (64, 512, 4096), (33, 200, 1024), (64, 4096, 4096), (16, 2048, 14336),
                                    # more tiles than SMs: a CTA's run crosses tile boundaries (partial first and last segments)
                                    (16, 25600, 512), (32, 20480, 1024), (8, 19000, 768),
                                    # narrow batches (the mma.sync kernel): K not a multiple of 256, ragged N, split tiles
                                    (4, 300, 320), (8, 128, 64), (7, 1000, 4096), (2, 19000, 1280)])
@pytest.mark.parametrize("bf", [False, True])
def test_gemm_w4a16_tensor_core(cuda, orc, M, N, K, bf):
    from nve_b200 import cuda_kernels as ck

    torch = cuda
    dt = torch.bfloat16 if bf else torch.float16
    nib, sc, X16, ref = _case(orc, M, N, K, 700 + M + N, bf)
    dx, dn, ds = dev(X16, dt), dev(nib), dev(sc)
    y32 = ck.gemm_w4a16(dx, dn, ds, N, K, out_dtype=torch.float32)
    torch.cuda.synchronize()
    assert ck.gemm_error() == 0
    # weights and scales are rounded to the activation type (as the reference dequantises to f16): ~2^-11 (f16)
    # or ~2^-8 (bf16) relative per weight; the f16 path stays far inside the stated tolerance, bf16 inside it
    assert rel_rms_err(y32.cpu().numpy(), ref) < 3e-3
    # the 16-bit output is the f32 accumulator rounded once (for bf16 that rounding alone is ~8e-3 of the RMS at
    # 4 sigma, so the tolerance is judged on the f32 output and the 16-bit output is checked as its rounding)
    y16 = ck.gemm_w4a16(dx, dn, ds, N, K)
    assert torch.equal(y16, y32.to(dt))
    if not bf:
        assert rel_rms_err(y16.float().cpu().numpy(), ref) < TOL
    # with a caller-provided workspace tiles are cut over K between CTAs: same result within f32 reassociation
    nbytes = ck.gemm_w4a16_scratch_bytes(M, N, K)
    if nbytes:
        scratch = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
        ys = ck.gemm_w4a16(dx, dn, ds, N, K, out_dtype=torch.float32, scratch=scratch)
        assert rel_rms_err(ys.cpu().numpy(), ref) < 3e-3
        assert ck.gemm_error() == 0


def test_gemm_matches_gemv_rows(cuda, orc):
    """Row m of the batched result equals the batch-1 W4A16 GEMV of row m within tolerance (different arithmetic:
    f16 weights on tensor cores vs the integer path)."""
    from nve_b200 import cuda_kernels as ck

    torch = cuda
    M, N, K = 16, 1024, 4096
    nib, sc, X16, ref = _case(orc, M, N, K, 801, False)
    dx, dn, ds = dev(X16, torch.float16), dev(nib), dev(sc)
    Y = ck.gemm_w4a16(dx, dn, ds, N, K, out_dtype=torch.float32).cpu().numpy()
    for m in (0, 7, 15):
        y = ck.matvec_w4a16_multi(dx[m].contiguous(), None, [(dn, ds, N)], K, out_dtype=torch.float32)[0].cpu().numpy().reshape(-1)
        assert rel_rms_err(Y[m], y) < 3e-3


@pytest.mark.parametrize("M,Ns,K", [(16, (4096, 1024, 1024), 4096), (8, (256, 128), 512), (64, (1024, 1000, 40), 1024),
                                     (8, (12800, 12864), 512)])
def test_gemm_multi_matrix_equals_single_calls(cuda, orc, M, Ns, K):
    """q/k/v (or gate/up) in one launch: same numbers as one call per matrix without a workspace, and within f32
    reassociation of them when the workspace lets the runs of the CTAs cut tiles (also across the matrices)."""
    from nve_b200 import cuda_kernels as ck

    torch = cuda
    X16 = orc.to_act16(orc.fill_normal(M * K, 950, 2)).reshape(M, K)
    dx = dev(X16, torch.float16)
    ws, singles = [], []
    for i, N in enumerate(Ns):
        nib, sc, _, _ = _case(orc, M, N, K, 960 + i, False)
        dn, ds = dev(nib), dev(sc)
        ws.append((dn, ds, N))
        singles.append(ck.gemm_w4a16(dx, dn, ds, N, K, out_dtype=torch.float32))
    outs = ck.gemm_w4a16_multi(dx, ws, K, out_dtype=torch.float32)
    for y, want in zip(outs, singles):
        assert torch.equal(y, want)
    scratch = torch.empty(ck.gemm_w4a16_multi_scratch_bytes(M, Ns, K), dtype=torch.uint8, device="cuda")
    outs = ck.gemm_w4a16_multi(dx, ws, K, out_dtype=torch.float32, scratch=scratch)
    for y, want in zip(outs, singles):
        assert rel_rms_err(y.cpu().numpy(), want.cpu().numpy()) < 1e-5
    outs16 = ck.gemm_w4a16_multi(dx, ws, K, scratch=scratch)
    for y16, y in zip(outs16, outs):
        assert torch.equal(y16, y.to(torch.float16))
    assert ck.gemm_error() == 0


def test_gemm_rejects_bad_arguments(cuda):
    from nve_b200 import _ffi
    from nve_b200 import cuda_kernels as ck

    torch = cuda
    x = torch.zeros((65, 64), dtype=torch.float16, device="cuda")
    nib = torch.zeros((128, 32), dtype=torch.uint8, device="cuda")
    sc = torch.zeros((128, 2), dtype=torch.float32, device="cuda")
    with pytest.raises(_ffi.NveKernelError):
        ck.gemm_w4a16(x, nib, sc, 128, 64)  # M > 64
    with pytest.raises(_ffi.NveKernelError):
        ck.gemm_w4a16(x[:8, :32].contiguous(), nib, sc, 128, 32)  # K % 64 != 0


@pytest.mark.parametrize("M", [1, 5, 64, 100, 130, 300])
@pytest.mark.parametrize("with_awq", [False, True])
def test_matmul_x_matches_q4_linear(cuda, orc, M, with_awq):
    """gpu_layer.matmul_x (the batch > 1 call site: GEMV at M == 1, the fused GEMM walked in 64-row slices up to
    128 rows, dequantisation + dense GEMM above)
    against the reference's CPU semantics q4_linear on the same 16-bit activations."""
    from nve_b200.gpu_layer import GpuW4, matmul_x

    torch = cuda
    N, K = 768, 2048
    W = orc.fill_normal(N * K, 931, 1, scale=0.02).reshape(N, K)
    blocks = orc.quantize_q4(W)
    nib, sc = orc.extract_for_gpu(blocks)
    awq = (0.5 + np.abs(orc.fill_normal(K, 931, 3))).astype(np.float32) if with_awq else None
    X16 = orc.to_act16(orc.fill_normal(M * K, 931, 2)).reshape(M, K)
    w = GpuW4(dev(nib), dev(sc), None if awq is None else dev(awq), N, K)
    y = matmul_x(dev(X16, torch.float16), w)
    assert tuple(y.shape) == (M, N)
    ref = orc.q4_linear(blocks, orc.from_act16(X16), awq_inv=awq)
    assert rel_rms_err(y.float().cpu().numpy(), ref) < TOL


def test_matmul_x_dense_route_bf16(cuda, orc):
    """Above 128 rows matmul_x dequantises to f16 and calls the dense GEMM; bf16 activations are converted to f16
    for it and the result is rounded to bf16 once (judged on the f32 reference within bf16's own rounding)."""
    from nve_b200.gpu_layer import DENSE_ROWS, GpuW4, matmul_x

    torch = cuda
    M, N, K = DENSE_ROWS + 72, 512, 1024
    nib, sc, X16, ref = _case(orc, M, N, K, 977, True)
    w = GpuW4(dev(nib), dev(sc), None, N, K)
    y = matmul_x(dev(X16, torch.bfloat16), w)
    assert y.dtype == torch.bfloat16 and tuple(y.shape) == (M, N)
    yf = y.float().cpu().numpy().astype(np.float64)
    rms = np.sqrt(np.mean(ref * ref))
    assert np.all(np.abs(yf - ref) <= np.abs(ref) * 2.0 ** -8 + 3e-3 * rms)  # half a bf16 ulp + the f16 GEMM's tolerance
    out = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    assert matmul_x(dev(X16, torch.bfloat16), w, out=out) is out
    assert torch.equal(out, y)


@pytest.mark.parametrize("kernel", ["mma", "tc"])
def test_gemm_parity_with_each_kernel_forced(cuda, kernel):
    """The library picks the kernel by batch size; NVE_B200_GEMM_KERNEL (read once per process) forces one.  The
    parity cases above are run again in a child process with each kernel forced, so that the mma.sync kernel is
    also checked at 16 and 32 batch rows and the tcgen05 kernel at 8 and fewer."""
    if os.environ.get("NVE_B200_GEMM_KERNEL_CHILD"):
        pytest.skip("already inside the forced-kernel child run")
    env = dict(os.environ, NVE_B200_GEMM_KERNEL=kernel, NVE_B200_GEMM_KERNEL_CHILD="1")
    res = subprocess.run([sys.executable, "-m", "pytest", os.path.abspath(__file__), "-q", "-x", "-m", "gpu", "-k",
                          "tensor_core or multi_matrix", "-p", "no:cacheprovider"],
                         env=env, capture_output=True, text=True, timeout=900, cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-2000:]
