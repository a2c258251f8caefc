"""GPU parity tests: every kernel of the decode path, called through the C ABI, against the CPU oracle.

Bars: int8 codes, activation scales, per-block integer dots, packed weights and every 16-bit result whose
arithmetic order the library fixes are compared bit for bit; W4A16 and final scaled outputs are additionally
held to max|y - ref| <= 1e-2 * RMS(ref) against the reference's CPU path (f32 accumulation).
"""
import numpy as np
import pytest

from helpers import TOL, dev, f16_bits, rel_rms_err, same_f16

pytestmark = pytest.mark.gpu

SHAPES = [(1, 32), (5, 64), (33, 416), (130, 1056), (512, 2048), (1024, 4096), (256, 14336), (96, 28672)]


def make_case(orc, N, K, seed, bf16=False):
    W = orc.fill_normal(N * K, seed, 1, scale=0.02).reshape(N, K)
    nib, sc = orc.extract_for_gpu(orc.quantize_q4(W))
    x16 = orc.to_act16(orc.fill_normal(K, seed, 2), bf16)
    return W, nib, sc, x16


# ------------------------------------------------------------------ activation quantizer
@pytest.mark.parametrize("tag,bf", [("f16", False), ("bf16", True)])
def test_quantize_q8_golden(cuda, orc, golden, tag, bf):
    from nve_b200 import cuda_kernels as ck

    torch = cuda
    x = dev(golden[f"act_{tag}"], torch.bfloat16 if bf else torch.float16)
    xq, xs = ck.quantize_q8(x)
    assert np.array_equal(xq.cpu().numpy(), golden[f"act_{tag}_q"])
    assert np.array_equal(xs.cpu().numpy().view(np.uint32), golden[f"act_{tag}_s"].view(np.uint32))


@pytest.mark.parametrize("K", [32, 2048, 4096, 8192, 14336, 28672])
def test_quantize_q8_random_bit_exact(cuda, orc, K):
    from nve_b200 import cuda_kernels as ck

    torch = cuda
    x16 = orc.to_act16(orc.fill_normal(K, 11, K) * 3.0)
    eq, es = orc.quantize_q8(x16)
    xq, xs = ck.quantize_f16_q8(dev(x16, torch.float16))  # the reference-signature entry point
    assert np.array_equal(xq.cpu().numpy(), eq)
    assert np.array_equal(xs.cpu().numpy().view(np.uint32), es.view(np.uint32))
    # a view that is only 2-byte aligned takes the scalar path and gives the same bits
    buf = torch.zeros(K + 8, dtype=torch.float16, device="cuda")
    buf[1:K + 1] = dev(x16, torch.float16)
    xq2, xs2 = ck.quantize_f16_q8(buf[1:K + 1])
    assert np.array_equal(xq2.cpu().numpy(), eq) and np.array_equal(xs2.cpu().numpy(), es)


# ------------------------------------------------------------------ W4A8
@pytest.mark.parametrize("N,K", SHAPES)
def test_w4a8_integer_dots_bit_exact(cuda, orc, N, K):
    from nve_b200 import cuda_kernels as ck

    _, nib, sc, x16 = make_case(orc, N, K, 100 + N)
    xq, xs = orc.quantize_q8(x16)
    I = ck.w4a8_idot(dev(xq), dev(nib), N, K)
    assert np.array_equal(I.cpu().numpy(), orc.w4a8_idot(xq, nib))


@pytest.mark.parametrize("N,K", SHAPES)
def test_w4a8_matvec(cuda, orc, N, K):
    from nve_b200 import cuda_kernels as ck

    torch = cuda
    _, nib, sc, x16 = make_case(orc, N, K, 200 + N)
    xq, xs = orc.quantize_q8(x16)
    dxq, dxs, dn, ds = dev(xq), dev(xs), dev(nib), dev(sc)
    # f32 output: the library's summation order is fixed, so the oracle restatement reproduces the bits
    y32 = ck.matvec_w4a8_multi(dxq, dxs, [(dn, ds, N)], K, out_dtype=torch.float32)[0].cpu().numpy().reshape(-1)
    exp32 = orc.w4a8_matvec_b200(xq, xs, nib, sc)
    assert np.array_equal(y32.view(np.uint32), exp32.view(np.uint32))
    # reference-signature entry point: f16(round) of the same value
    y16 = ck.matvec_w4a8(dxq, dxs, dn, ds, N, K)
    assert np.array_equal(f16_bits(y16).reshape(-1), orc.f32_to_f16_bits(exp32))
    # and within tolerance of the exact sum
    assert rel_rms_err(y32, orc.w4a8_matvec_f64(xq, xs, nib, sc)) < 1e-5
    assert rel_rms_err(y16.float().cpu().numpy(), orc.w4a8_matvec_f64(xq, xs, nib, sc)) < TOL


def test_w4a8_golden(cuda, orc, golden):
    from nve_b200 import cuda_kernels as ck

    torch = cuda
    g = golden
    N, K = g["g_nibbles"].shape[0], g["g_xq"].size
    y = ck.matvec_w4a8_multi(dev(g["g_xq"]), dev(g["g_xs"]), [(dev(g["g_nibbles"]), dev(g["g_scales"]), N)], K,
                             out_dtype=torch.float32)[0].cpu().numpy().reshape(-1)
    assert np.array_equal(y.view(np.uint32), g["g_y_w4a8_b200"].view(np.uint32))
    I = ck.w4a8_idot(dev(g["g_xq"]), dev(g["g_nibbles"]), N, K)
    assert np.array_equal(I.cpu().numpy(), g["g_idot"])


# ------------------------------------------------------------------ W4A16
@pytest.mark.parametrize("N,K", SHAPES)
@pytest.mark.parametrize("bf", [False, True])
def test_w4a16_matvec(cuda, orc, N, K, bf):
    from nve_b200 import cuda_kernels as ck

    torch = cuda
    W, nib, sc, x16 = make_case(orc, N, K, 300 + N, bf)
    dx = dev(x16, torch.bfloat16 if bf else torch.float16)
    dn, ds = dev(nib), dev(sc)
    y32 = ck.matvec_w4a16_multi(dx, None, [(dn, ds, N)], K, out_dtype=torch.float32)[0].cpu().numpy().reshape(-1)
    exp32 = orc.w4a16_matvec_b200(x16, nib, sc, bf16=bf)
    assert np.array_equal(y32.view(np.uint32), exp32.view(np.uint32))
    # the oracle that decides parity: the reference CPU path on the same 16-bit-rounded activations
    xf = orc.from_act16(x16, bf)
    cpu = orc.q4_matvec(orc.quantize_q4(W), xf, order="scalar")
    assert rel_rms_err(y32, cpu) < 1e-3
    out16 = ck.matvec_w4a16_multi(dx, None, [(dn, ds, N)], K, out_dtype=dx.dtype)[0]
    assert rel_rms_err(out16.float().cpu().numpy(), cpu) < TOL


def test_w4a16_reference_entry_points(cuda, orc, golden):
    from nve_b200 import cuda_kernels as ck

    torch = cuda
    g = golden
    N, K = g["g_nibbles"].shape[0], g["g_x16"].size
    dx = dev(g["g_x16"], torch.float16).view(1, K)
    y = ck.fused_matvec_w4a16(dx, dev(g["g_nibbles"]), dev(g["g_scales"]), None, N, K)
    # row 6 holds weights near the f32 maximum: its scaled sum overflows to NaN on host and device alike
    assert same_f16(f16_bits(y), orc.f32_to_f16_bits(g["g_y_w4a16_b200"]))
    fin = np.isfinite(g["g_y_cpu_scalar"]) & np.isfinite(g["g_y_w4a16_b200"])
    assert fin.sum() >= N - 1
    assert rel_rms_err(y.float().cpu().numpy().reshape(-1)[fin], g["g_y_cpu_scalar"][fin]) < TOL
    # AWQ: x is multiplied by the inverse scales before the dot (weights were quantised pre-scaled)
    ya = ck.fused_matvec_w4a16(dx, dev(g["g_awq_nibbles"]), dev(g["g_awq_scales"]), dev(g["g_awq_inv"]), N, K)
    assert same_f16(f16_bits(ya), orc.f32_to_f16_bits(g["g_y_awq_b200"]))
    fin = np.isfinite(g["g_y_awq_cpu_scalar"]) & np.isfinite(g["g_y_awq_b200"])
    assert fin.sum() >= N - 1
    assert rel_rms_err(ya.float().cpu().numpy().reshape(-1)[fin], g["g_y_awq_cpu_scalar"][fin]) < TOL
    # q/k/v in one launch equals three launches
    n1, n2 = 32, 16
    nib, sc = dev(g["g_nibbles"]), dev(g["g_scales"])
    parts = [(nib[:n1].contiguous(), sc[:n1].contiguous(), n1), (nib[n1:n1 + n2].contiguous(), sc[n1:n1 + n2].contiguous(), n2),
             (nib[n1 + n2:].contiguous(), sc[n1 + n2:].contiguous(), N - n1 - n2)]
    q, k, v = ck.fused_qkv_matvec_w4a16(dx, parts[0][0], parts[0][1], None, n1, parts[1][0], parts[1][1], None, n2,
                                        parts[2][0], parts[2][1], None, N - n1 - n2, K)
    joined = torch.cat([q, k, v], dim=1)
    assert same_f16(f16_bits(joined), f16_bits(y))


def test_config1_w4a16_up_proj(cuda, orc, golden):
    """Measurement configuration 1: x [1x2048], W [8192x2048] ~N(0,0.02) through the reference quantizer, y [1x8192]."""
    import hashlib

    from nve_b200 import cuda_kernels as ck

    torch = cuda
    seed = int(golden["seed"][0])
    W = orc.fill_normal(8192 * 2048, seed, 10, scale=0.02).reshape(8192, 2048)
    x16 = orc.to_act16(orc.fill_normal(2048, seed, 11))
    # weights prepared on the device: bit-identical to quantize_block_q4 + extract_for_gpu
    nib, sc = ck.q4_quantize(dev(W))
    sha = lambda a: np.frombuffer(hashlib.sha256(a.tobytes()).digest(), np.uint8)
    assert np.array_equal(sha(nib.cpu().numpy()), golden["c1_nibbles_sha"])
    assert np.array_equal(sha(sc.cpu().numpy()), golden["c1_scales_sha"])
    y32 = ck.matvec_w4a16_multi(dev(x16, torch.float16), None, [(nib, sc, 8192)], 2048, out_dtype=torch.float32)[0]
    y32 = y32.cpu().numpy().reshape(-1)
    assert np.array_equal(sha(y32), golden["c1_y_b200_sha"])
    cpu = orc.q4_matvec(orc.quantize_q4(W), orc.from_act16(x16))
    assert np.array_equal(sha(cpu), golden["c1_y_cpu_scalar_sha"])
    assert rel_rms_err(y32, cpu) < 1e-3
    y16 = ck.fused_matvec_w4a16(dev(x16, torch.float16).view(1, -1), nib, sc, None, 8192, 2048)
    assert rel_rms_err(y16.float().cpu().numpy(), cpu) < TOL


def test_multi_matrix_and_residual_epilogue(cuda, orc):
    from nve_b200 import cuda_kernels as ck

    torch = cuda
    K = 2048
    mats = []
    for i, N in enumerate((2048, 512, 512)):
        _, nib, sc, _ = make_case(orc, N, K, 400 + i)
        mats.append((dev(nib), dev(sc), N))
    x16 = orc.to_act16(orc.fill_normal(K, 400, 9))
    xq, xs = orc.quantize_q8(x16)
    dxq, dxs, dx = dev(xq), dev(xs), dev(x16, torch.float16)
    fused = ck.matvec_w4a8_multi(dxq, dxs, mats, K)
    for m, y in zip(mats, fused):
        assert torch.equal(y, ck.matvec_w4a8(dxq, dxs, m[0], m[1], m[2], K))
    fused16 = ck.matvec_w4a16_multi(dx, None, mats, K)
    for m, y in zip(mats, fused16):
        assert torch.equal(y, ck.fused_matvec_w4a16(dx, m[0], m[1], None, m[2], K))
    # residual in the epilogue == GEMV then nve_add_inplace_f16
    res = dev(orc.to_act16(orc.fill_normal(2048, 401, 1)), torch.float16).view(1, -1)
    y = ck.matvec_w4a8_multi(dxq, dxs, [mats[0]], K, residuals=[res])[0]
    ref = res.clone()
    ck.add_inplace(ref, fused[0])
    assert torch.equal(y, ref)
    # in place (out aliases residual), as the captured graph uses it
    h = res.clone()
    ck.matvec_w4a16_multi(dx, None, [mats[0]], K, outs=[h], residuals=[h])
    ref2 = res.clone()
    ck.add_inplace(ref2, fused16[0])
    assert torch.equal(h, ref2)


def test_unaligned_weight_view_uses_generic_path(cuda, orc):
    from nve_b200 import cuda_kernels as ck

    torch = cuda
    N, K = 40, 256
    _, nib, sc, x16 = make_case(orc, N, K, 500)
    xq, xs = orc.quantize_q8(x16)
    buf = torch.zeros(N * K // 2 + 64, dtype=torch.uint8, device="cuda")
    view = buf[2:2 + N * K // 2]
    view.copy_(dev(nib).view(-1))
    y = ck.matvec_w4a8(dev(xq), dev(xs), view.view(N, K // 2), dev(sc), N, K)
    assert np.array_equal(f16_bits(y).reshape(-1), orc.f32_to_f16_bits(orc.w4a8_matvec_b200(xq, xs, nib, sc)))
    y2 = ck.fused_matvec_w4a16(dev(x16, torch.float16), view.view(N, K // 2), dev(sc), None, N, K)
    assert np.array_equal(f16_bits(y2).reshape(-1), orc.f32_to_f16_bits(orc.w4a16_matvec_b200(x16, nib, sc)))


def test_bad_shapes_are_rejected(cuda):
    from nve_b200 import _ffi
    from nve_b200 import cuda_kernels as ck

    torch = cuda
    x = torch.zeros(48, dtype=torch.float16, device="cuda")
    with pytest.raises(ValueError):
        ck.quantize_f16_q8(x)
    nib = torch.zeros((4, 24), dtype=torch.uint8, device="cuda")
    sc = torch.zeros((4, 2), dtype=torch.float32, device="cuda")
    with pytest.raises(_ffi.NveKernelError):
        ck.fused_matvec_w4a16(x, nib, sc, None, 4, 48)


# ------------------------------------------------------------------ full-size properties (Llama-3.1-8B shapes)
def test_full_size_properties_8b_gate(cuda, orc):
    """14336 x 4096 (8B gate/up): sampled rows against the oracle, exact homogeneity, zero input."""
    from nve_b200 import cuda_kernels as ck

    torch = cuda
    N, K = 14336, 4096
    W = ck.fill_normal(N * K, 7, 1, scale=0.02).view(N, K)
    nib, sc = ck.q4_quantize(W)
    x16 = orc.to_act16(orc.fill_normal(K, 7, 2))
    dx = dev(x16, torch.float16)
    xq, xs = ck.quantize_f16_q8(dx)
    y8 = ck.matvec_w4a8_multi(xq, xs, [(nib, sc, N)], K, out_dtype=torch.float32)[0].view(-1)
    y16 = ck.matvec_w4a16_multi(dx, None, [(nib, sc, N)], K, out_dtype=torch.float32)[0].view(-1)
    rows = np.unique(np.concatenate([[0, 1, 2, 3, N - 1, N - 2], np.random.default_rng(0).integers(0, N, 120)]))
    nib_s, sc_s = nib[rows].cpu().numpy(), sc[rows].cpu().numpy()
    exq, exs = orc.quantize_q8(x16)
    assert np.array_equal(xq.cpu().numpy(), exq)
    assert np.array_equal(y8[rows].cpu().numpy().view(np.uint32), orc.w4a8_matvec_b200(exq, exs, nib_s, sc_s).view(np.uint32))
    assert np.array_equal(y16[rows].cpu().numpy().view(np.uint32), orc.w4a16_matvec_b200(x16, nib_s, sc_s).view(np.uint32))
    # device-quantised weights equal the oracle's for the sampled rows (the generator is shared)
    Ws = np.stack([orc.fill_normal(K, 7, 1, first=int(r) * K, scale=0.02) for r in rows])
    en, es = orc.extract_for_gpu(orc.quantize_q4(Ws))
    assert np.array_equal(nib_s, en) and np.array_equal(sc_s.view(np.uint32), es.view(np.uint32))
    # scaling x by 2 scales every group amax by 2: identical codes, outputs exactly doubled
    dx2 = (dx.float() * 2).half()
    y16b = ck.matvec_w4a16_multi(dx2, None, [(nib, sc, N)], K, out_dtype=torch.float32)[0].view(-1)
    assert torch.equal(y16b, y16 * 2)
    z = torch.zeros_like(dx)
    assert torch.count_nonzero(ck.matvec_w4a16_multi(z, None, [(nib, sc, N)], K, out_dtype=torch.float32)[0]) == 0
    # a checksum of all integer dots: sum_n I[n, b] = (sum_n q[n, b, :]) . xq[b, :]
    I = ck.w4a8_idot(xq, nib, N, K).to(torch.int64).sum(0).cpu().numpy()
    from oracle import np_oracle as npo
    step = 1024
    colsum = np.zeros(K, np.int64)
    for r0 in range(0, N, step):
        colsum += npo.unpack_gpu(nib[r0:r0 + step].cpu().numpy()).astype(np.int64).sum(0)
    assert np.array_equal(I, (colsum * exq.astype(np.int64)).reshape(K // 32, 32).sum(1))


# ------------------------------------------------------------------ weights
def test_q4_quantize_and_repack_bit_exact(cuda, orc, golden):
    from nve_b200 import cuda_kernels as ck

    torch = cuda
    nib, sc = ck.q4_quantize(dev(golden["w_edge"]))
    assert np.array_equal(nib.cpu().numpy(), golden["w_edge_nibbles"])
    assert np.array_equal(sc.cpu().numpy().view(np.uint32), golden["w_edge_scales"].view(np.uint32))
    n2, s2 = ck.q4_repack_blocks(dev(golden["w_edge_blocks"]).view(-1), 16, 128)
    assert np.array_equal(n2.cpu().numpy(), golden["w_edge_nibbles"])
    assert np.array_equal(s2.cpu().numpy().view(np.uint32), golden["w_edge_scales"].view(np.uint32))
    # AWQ pre-scaling
    na, sa = ck.q4_quantize(dev(golden["g_w"]), dev(golden["g_awq"]))
    assert np.array_equal(na.cpu().numpy(), golden["g_awq_nibbles"])
    assert np.array_equal(sa.cpu().numpy().view(np.uint32), golden["g_awq_scales"].view(np.uint32))
    rng = np.random.default_rng(9)
    W = (rng.standard_normal((257, 320)) * rng.choice([1e-3, 0.02, 1.0, 50.0], (257, 1))).astype(np.float32)
    en, es = orc.extract_for_gpu(orc.quantize_q4(W))
    dn, ds = ck.q4_quantize(dev(W))
    assert np.array_equal(dn.cpu().numpy(), en) and np.array_equal(ds.cpu().numpy().view(np.uint32), es.view(np.uint32))


@pytest.mark.parametrize("bf", [False, True])
def test_dequant_bit_exact(cuda, orc, golden, bf):
    from nve_b200 import cuda_kernels as ck

    torch = cuda
    g = golden
    N, K = g["g_nibbles"].shape[0], g["g_x16"].size
    out = ck.dequant_w4a16_any(dev(g["g_nibbles"]), dev(g["g_scales"]), None, N, K, torch.bfloat16 if bf else torch.float16)
    assert same_f16(f16_bits(out), orc.dequant_w4a16(g["g_nibbles"], g["g_scales"], None, bf), bf)
    if not bf:
        out2 = ck.dequant_w4a16(dev(g["g_awq_nibbles"]), dev(g["g_awq_scales"]), dev(g["g_awq_inv"]), N, K)
        # the pre-scaled near-maximum row overflows: scale inf, codes 0, dequantised value NaN on both sides
        assert same_f16(f16_bits(out2), orc.dequant_w4a16(g["g_awq_nibbles"], g["g_awq_scales"], g["g_awq_inv"]))


def test_generator_bit_exact(cuda, orc):
    from nve_b200 import cuda_kernels as ck

    torch = cuda
    a = ck.fill_normal(10000, 99, 4, first=123, scale=0.02).cpu().numpy()
    assert np.array_equal(a.view(np.uint32), orc.fill_normal(10000, 99, 4, first=123, scale=0.02).view(np.uint32))
    h = ck.fill_normal(4096, 99, 5, dtype=torch.float16)
    assert np.array_equal(f16_bits(h), orc.to_act16(orc.fill_normal(4096, 99, 5)))


def test_matvec_f16_dense(cuda, orc):
    from nve_b200 import cuda_kernels as ck

    torch = cuda
    N, K = 300, 1024
    W = orc.fill_normal(N * K, 3, 1, scale=0.02).reshape(N, K)
    x = orc.fill_normal(K, 3, 2)
    W16, x16 = orc.to_act16(W), orc.to_act16(x)
    y = ck.fused_matvec(dev(x16, torch.float16), dev(W16, torch.float16), N, K)
    ref = orc.from_act16(W16).astype(np.float64) @ orc.from_act16(x16).astype(np.float64)
    assert rel_rms_err(y.float().cpu().numpy(), ref) < 2e-3


# ------------------------------------------------------------------ AWQ multiplier folded into the W4A8 quantiser
@pytest.mark.parametrize("bf", [False, True])
def test_quantize_q8_awq_bit_exact_and_fused_prologue(cuda, orc, bf):
    """codes / scales of x * awq_inv equal the oracle bit for bit; the fused RMSNorm + W4A8 GEMV with the multiplier
    equals RMSNorm -> quantize_q8_awq -> W4A8 GEMV bit for bit."""
    from nve_b200 import cuda_kernels as ck

    torch = cuda
    dt = torch.bfloat16 if bf else torch.float16
    K, N = 4096, 512
    x16 = orc.to_act16(orc.fill_normal(K, 611, 1) * 2.0, bf)
    awq = (1.0 / (0.25 + np.abs(orc.fill_normal(K, 611, 2)))).astype(np.float32)  # 0.2 .. 4, a few large
    awq[7] = 1.0e3
    xq, xs = ck.quantize_q8_awq(dev(x16, dt), dev(awq))
    eq, es = orc.quantize_q8_awq(x16, awq, bf)
    assert np.array_equal(xq.cpu().numpy(), eq)
    assert np.array_equal(xs.cpu().numpy(), es)
    W = orc.fill_normal(N * K, 611, 3, scale=0.02).reshape(N, K)
    nib, sc = orc.extract_for_gpu(orc.quantize_q4(W))
    mats = [(dev(nib), dev(sc), N)]
    nw = dev(orc.to_act16(1.0 + 0.1 * orc.fill_normal(K, 611, 4), bf), dt)
    h = dev(x16, dt).view(1, -1)
    normed = ck.rms_norm(h, nw, 1e-5)
    q2, s2 = ck.quantize_q8_awq(normed, dev(awq))
    sep = ck.matvec_w4a8_multi(q2, s2, mats, K, out_dtype=torch.float32)[0]
    fused = ck.rmsnorm_matvec_w4a8_awq_multi(h, nw, 1e-5, dev(awq), mats, K, out_dtype=torch.float32)[0]
    assert torch.equal(sep, fused)


# ------------------------------------------------------------------ W4A16 fixed point under hostile dynamic ranges
@pytest.mark.parametrize("case", ["outlier", "tiny", "awq_large"])
def test_w4a16_fixed_point_hostile_ranges(cuda, orc, case):
    """The W4A16 GEMV carries the activations as per-block 16-bit fixed point (step amax/32767).  Where that differs
    most from per-element f16 -- one 1e4x outlier per block, values near the f16 subnormal range, a large AWQ
    multiplier -- the result must still be within 1e-2 of the output RMS of the reference's f32 row dot
    (q4_dot_row_scalar on the same 16-bit activations)."""
    from nve_b200 import cuda_kernels as ck

    torch = cuda
    N, K = 1024, 4096
    x = orc.fill_normal(K, 621, 1)
    awq = None
    if case == "outlier":
        x = x * 1.0e-3
        x[5::32] = 10.0  # one element 1e4 x its block-mates
    elif case == "tiny":
        x = x * 6.0e-5   # f16 subnormals and the smallest normals
    else:
        awq = (1.0 + np.abs(orc.fill_normal(K, 621, 3))).astype(np.float32)
        awq[11::64] = 1.0e3
    x16 = orc.to_act16(x)
    W = orc.fill_normal(N * K, 621, 2, scale=0.02).reshape(N, K)
    blocks = orc.quantize_q4(W)
    nib, sc = orc.extract_for_gpu(blocks)
    y = ck.matvec_w4a16_multi(dev(x16, torch.float16).view(1, -1), None if awq is None else dev(awq), [(dev(nib), dev(sc), N)], K,
                              out_dtype=torch.float32)[0]
    ref = orc.q4_matvec(blocks, orc.from_act16(x16), awq_inv=awq)
    assert np.all(np.isfinite(y.cpu().numpy()))
    assert rel_rms_err(y.cpu().numpy(), ref) < TOL
