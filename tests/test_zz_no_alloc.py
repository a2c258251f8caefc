"""GPU: the allocation-free batched GEMM entry point (nve_b200_gemm_w4a16_noalloc).

Some callers of the batched GEMM have nowhere to get a workspace from: the reference's batch > 1 call site only
holds activation and weight tensors, and it may run while a CUDA graph is being captured, when device allocation
is forbidden.  For them the library keeps the partial sums of tiles that several CTAs share in a fixed array of its own.  This file checks,
through the C ABI, that the entry point gives the same result as the ordinary one (which takes a caller-provided
workspace) on two calls in a row -- the second with different inputs, so stale partials from the first call
would show -- and that a shape whose partials exceed the fixed array is refused.  It is collected last so that a
run that stops at the first failure has already executed every other test."""
import numpy as np
import pytest

from helpers import dev, rel_rms_err

pytestmark = pytest.mark.gpu


def _inputs(orc, M, N, K, seed):
    W = orc.fill_normal(N * K, seed, 1, scale=0.02).reshape(N, K)
    nib, sc = orc.extract_for_gpu(orc.quantize_q4(W))
    X16 = orc.to_act16(orc.fill_normal(M * K, seed, 2)).reshape(M, K)
    return nib, sc, X16


def test_noalloc_gemm_matches_workspace_gemm_twice(cuda, orc):
    from nve_b200 import cuda_kernels as ck

    torch = cuda
    M, N, K = 32, 1024, 4096  # 8 weight tiles, each cut over K between 8 CTAs: the workspace is really used
    assert ck.gemm_w4a16_scratch_bytes(M, N, K) > 0
    for call, seed in enumerate((911, 912)):
        nib, sc, X16 = _inputs(orc, M, N, K, seed)
        dx, dn, ds = dev(X16, torch.float16), dev(nib), dev(sc)
        scratch = torch.empty(ck.gemm_w4a16_scratch_bytes(M, N, K), dtype=torch.uint8, device="cuda")
        want = ck.gemm_w4a16(dx, dn, ds, N, K, out_dtype=torch.float32, scratch=scratch)
        got = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
        before = torch.cuda.memory_allocated()
        ck.gemm_w4a16_noalloc(dx, dn, ds, N, K, got)
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before  # nothing was allocated through torch either
        assert ck.gemm_error() == 0
        assert rel_rms_err(got.cpu().numpy(), want.cpu().numpy()) < 3e-3, f"call {call}"
        assert torch.equal(got, want), f"call {call}: same kernels, same split, same summation order"
        # 16-bit output form
        got16 = torch.empty((M, N), dtype=torch.float16, device="cuda")
        ck.gemm_w4a16_noalloc(dx, dn, ds, N, K, got16)
        assert torch.equal(got16, want.to(torch.float16))


def test_noalloc_gemm_bf16_input_and_exact_limit(cuda, orc):
    """bf16 activations (their f16 copy then shares the fixed array with the partial sums) and a shape whose workspace
    is exactly the 4 MiB limit: both must equal the workspace form bit for bit."""
    from nve_b200 import cuda_kernels as ck

    torch = cuda
    for (M, N, K, dt, bf) in ((16, 1024, 4096, torch.bfloat16, True), (64, 1024, 4096, torch.float16, False)):
        W = orc.fill_normal(N * K, 921, 1, scale=0.02).reshape(N, K)
        nib, sc = orc.extract_for_gpu(orc.quantize_q4(W))
        X16 = orc.to_act16(orc.fill_normal(M * K, 921, 2), bf).reshape(M, K)
        dx, dn, ds = dev(X16, dt), dev(nib), dev(sc)
        nbytes = ck.gemm_w4a16_scratch_bytes(M, N, K)
        if not bf:
            # 64 CTAs x 2 partial tiles x 64 x 128 floats = exactly the fixed 4 MiB array (the workspace form also
            # reserves room for a 16-bit copy of the activations, which f16 input does not use)
            assert nbytes - M * K * 2 == 4 * 1024 * 1024
        scratch = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
        want = ck.gemm_w4a16(dx, dn, ds, N, K, out_dtype=torch.float32, scratch=scratch)
        for _call in range(2):
            got = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
            ck.gemm_w4a16_noalloc(dx, dn, ds, N, K, got)
            torch.cuda.synchronize()
            assert ck.gemm_error() == 0
            assert torch.equal(got, want)


def test_noalloc_gemm_refuses_oversized_workspace(cuda):
    from nve_b200 import _ffi
    from nve_b200 import cuda_kernels as ck

    torch = cuda
    M, N, K = 64, 2048, 4096  # 128 CTAs x 2 partial tiles x 64 x 128 floats = 8 MiB > the fixed 4 MiB
    assert ck.gemm_w4a16_scratch_bytes(M, N, K) > 4 * 1024 * 1024
    x = torch.zeros((M, K), dtype=torch.float16, device="cuda")
    nib = torch.zeros((N, K // 2), dtype=torch.uint8, device="cuda")
    sc = torch.zeros((N, K // 32), dtype=torch.float32, device="cuda")
    out = torch.empty((M, N), dtype=torch.float16, device="cuda")
    with pytest.raises(_ffi.NveKernelError) as ei:
        ck.gemm_w4a16_noalloc(x, nib, sc, N, K, out)
    assert ei.value.status == 5  # NVE_ERR_TOO_LARGE
