"""GPU parity tests for the activation-side and attention-side kernels, the decode layer and the graph."""
import numpy as np
import pytest

from helpers import TOL, dev, f16_bits, rel_rms_err

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n", [32, 64, 2048, 4096, 8192, 14336])
@pytest.mark.parametrize("bf", [False, True])
def test_rms_norm_bit_exact_and_fused_quantize(cuda, orc, n, bf):
    from nve_b200 import cuda_kernels as ck

    torch = cuda
    dt = torch.bfloat16 if bf else torch.float16
    x16 = orc.to_act16(orc.fill_normal(n, 21, n) * 1.7, bf)
    w16 = orc.to_act16(1.0 + 0.1 * orc.fill_normal(n, 22, n), bf)
    exp = orc.rms_norm_16(x16, w16, 1e-5, bf)
    dx, dw = dev(x16, dt), dev(w16, dt)
    out = ck.rms_norm(dx, dw, 1e-5)
    assert np.array_equal(f16_bits(out), exp)
    # against the reference CPU form (f64 accumulation): one 16-bit rounding apart
    ref = orc.rms_norm_f64(orc.from_act16(x16, bf), orc.from_act16(w16, bf), 1e-5)
    assert rel_rms_err(out.float().cpu().numpy(), ref) < (2e-2 if bf else 3e-3)
    # fused RMSNorm -> quantise == the two launches of the reference call site
    xq, xs, normed = ck.rmsnorm_quantize_q8(dx, dw, 1e-5, want_normed=True)
    eq, es = orc.quantize_q8(exp, bf)
    assert np.array_equal(f16_bits(normed), exp)
    assert np.array_equal(xq.cpu().numpy(), eq) and np.array_equal(xs.cpu().numpy().view(np.uint32), es.view(np.uint32))
    if not bf:
        out2 = ck.fused_rms_norm(dx, dw, 1e-5)  # reference-signature entry point
        assert torch.equal(out2, out)


def test_rms_norm_ragged_length(cuda, orc):
    from nve_b200 import cuda_kernels as ck

    torch = cuda
    n = 1000 + 3
    x16 = orc.to_act16(orc.fill_normal(n, 23, 1))
    w16 = orc.to_act16(np.ones(n, np.float32))
    out = ck.fused_rms_norm(dev(x16, torch.float16), dev(w16, torch.float16), 1e-5)
    assert np.array_equal(f16_bits(out), orc.rms_norm_16(x16, w16, 1e-5))


@pytest.mark.parametrize("n", [64, 8192, 14336])
def test_silu_mul_and_fused_quantize(cuda, orc, n):
    from nve_b200 import cuda_kernels as ck

    torch = cuda
    g16 = orc.to_act16(orc.fill_normal(n, 31, 1) * 2.0)
    u16 = orc.to_act16(orc.fill_normal(n, 31, 2))
    exp = orc.from_act16(orc.silu_mul_16(g16, u16))
    gate = dev(g16, torch.float16)
    up = dev(u16, torch.float16)
    got = gate.clone()
    ck.silu_mul_inplace(got, up)
    # expf differs in the last place between host and device libm: allow one f16 ulp of the result
    gotf = got.float().cpu().numpy()
    assert np.all(np.abs(gotf - exp) <= np.maximum(np.abs(exp) * 2.0**-10, 2.0**-24))
    assert np.mean(f16_bits(got) == orc.to_act16(exp)) > 0.99
    # fused silu*up -> quantise == silu_mul then quantize on the same device values
    xq, xs, mid = ck.silu_mul_quantize_q8(gate, up, want_mid=True)
    assert torch.equal(mid, got)
    eq, es = orc.quantize_q8(f16_bits(got))
    assert np.array_equal(xq.cpu().numpy(), eq) and np.array_equal(xs.cpu().numpy().view(np.uint32), es.view(np.uint32))


@pytest.mark.parametrize("n,N,use_awq", [(64, 40, False), (8192, 256, True), (14336, 512, False)])
def test_silu_mul_x16_planes_feed_the_w4a16_gemv(cuda, orc, n, N, use_awq):
    """silu*up -> fixed-point planes in one launch: the planes equal the oracle's fixed-point codes of the device's
    own silu*up values, and the GEMV fed with them is bit-identical to the GEMV fed with the 16-bit values."""
    from nve_b200 import cuda_kernels as ck

    torch = cuda
    g16 = orc.to_act16(orc.fill_normal(n, 41, 1) * 2.0)
    u16 = orc.to_act16(orc.fill_normal(n, 41, 2))
    gate, up = dev(g16, torch.float16), dev(u16, torch.float16)
    awq_np = (0.5 + np.abs(orc.fill_normal(n, 41, 3))).astype(np.float32) if use_awq else None
    awq = dev(awq_np) if use_awq else None
    mid_ref = gate.clone()
    ck.silu_mul_inplace(mid_ref, up)
    x_lo, x_hi, xs, mid = ck.silu_mul_x16(gate, up, awq, want_mid=True)
    assert torch.equal(mid, mid_ref)
    codes, scales = orc.x16_fixedpoint(f16_bits(mid_ref), False, awq_np)
    got = x_lo.cpu().numpy().astype(np.int32) + 256 * x_hi.cpu().numpy().astype(np.int32)
    assert np.array_equal(got, codes)
    assert np.array_equal(xs.cpu().numpy().view(np.uint32), scales.view(np.uint32))
    # the GEMV from planes == the GEMV from the 16-bit vector (same kernel arithmetic after staging)
    W = orc.fill_normal(N * n, 42, 1, scale=0.02).reshape(N, n)
    nib, sc = orc.extract_for_gpu(orc.quantize_q4(W))
    dn, ds = dev(nib), dev(sc)
    res = dev(orc.to_act16(orc.fill_normal(N, 42, 9)), torch.float16).view(1, N)
    y_ref = ck.matvec_w4a16_multi(mid_ref.view(-1), awq, [(dn, ds, N)], n, out_dtype=torch.float32)[0]
    y_pl = ck.matvec_w4a16_planes_multi(x_lo, x_hi, xs, [(dn, ds, N)], n, out_dtype=torch.float32)[0]
    assert torch.equal(y_ref, y_pl)
    o_ref = ck.matvec_w4a16_multi(mid_ref.view(-1), awq, [(dn, ds, N)], n, residuals=[res])[0]
    o_pl = ck.matvec_w4a16_planes_multi(x_lo, x_hi, xs, [(dn, ds, N)], n, residuals=[res])[0]
    assert torch.equal(o_ref, o_pl)


def test_add_inplace_and_layer_norm(cuda, orc):
    from nve_b200 import cuda_kernels as ck

    torch = cuda
    n = 4096
    a16, b16 = orc.to_act16(orc.fill_normal(n, 41, 1)), orc.to_act16(orc.fill_normal(n, 41, 2))
    a = dev(a16, torch.float16)
    ck.add_inplace(a, dev(b16, torch.float16))
    assert np.array_equal(f16_bits(a), orc.to_act16(orc.from_act16(a16) + orc.from_act16(b16)))
    x = orc.from_act16(a16).astype(np.float64)
    w = orc.from_act16(b16).astype(np.float64)
    ln = (x - x.mean()) / np.sqrt(x.var() + 1e-5) * w + 0.25
    bias = torch.full((n,), 0.25, dtype=torch.float16, device="cuda")
    out = ck.fused_layer_norm(dev(a16, torch.float16), dev(b16, torch.float16), bias, 1e-5)
    assert rel_rms_err(out.float().cpu().numpy(), ln) < 5e-3


def _rope_tables(orc, torch, hd, max_seq, theta=10000.0):
    cos, sin = orc.rope_tables_f32(hd, max_seq, theta)
    c16, s16 = orc.to_act16(cos), orc.to_act16(sin)
    return c16, s16, dev(c16, torch.float16), dev(s16, torch.float16)


@pytest.mark.parametrize("nh,nkv,hd", [(32, 8, 64), (32, 8, 128), (64, 8, 128)])
def test_rope_variants_bit_exact(cuda, orc, nh, nkv, hd):
    from nve_b200 import cuda_kernels as ck

    torch = cuda
    max_seq, pos = 64, 37
    c16, s16, dc, ds = _rope_tables(orc, torch, hd, max_seq)
    q16 = orc.to_act16(orc.fill_normal(nh * hd, 51, 1))
    k16 = orc.to_act16(orc.fill_normal(nkv * hd, 51, 2))
    cr, sr = orc.from_act16(c16[pos]), orc.from_act16(s16[pos])
    eq = orc.to_act16(orc.rope_apply(orc.from_act16(q16), nh, hd, cr, sr))
    ek = orc.to_act16(orc.rope_apply(orc.from_act16(k16), nkv, hd, cr, sr))
    q, k = dev(q16, torch.float16).view(nh, hd), dev(k16, torch.float16).view(nkv, hd)
    ck.fused_rope_decode(q, k, dc[pos].contiguous(), ds[pos].contiguous(), nh, nkv, hd)
    assert np.array_equal(f16_bits(q), eq) and np.array_equal(f16_bits(k), ek)
    q2, k2 = dev(q16, torch.float16).view(nh, hd), dev(k16, torch.float16).view(nkv, hd)
    d_pos = torch.tensor([pos], dtype=torch.int32, device="cuda")
    ck.rope_decode_dyn_inplace(q2, k2, dc, ds, nh, nkv, hd, d_pos.data_ptr())
    assert torch.equal(q2, q) and torch.equal(k2, k)
    # prefill: 3 tokens starting at position 5
    T, start = 3, 5
    qp16 = orc.to_act16(orc.fill_normal(T * nh * hd, 52, 1))
    kp16 = orc.to_act16(orc.fill_normal(T * nkv * hd, 52, 2))
    qp, kp = dev(qp16, torch.float16).view(T, nh, hd), dev(kp16, torch.float16).view(T, nkv, hd)
    ck.fused_rope_prefill(qp, kp, dc, ds, T, nh, nkv, hd, start)
    for t in range(T):
        cr, sr = orc.from_act16(c16[start + t]), orc.from_act16(s16[start + t])
        e = orc.to_act16(orc.rope_apply(orc.from_act16(qp16.reshape(T, -1)[t]), nh, hd, cr, sr))
        assert np.array_equal(f16_bits(qp[t]), e)
        e = orc.to_act16(orc.rope_apply(orc.from_act16(kp16.reshape(T, -1)[t]), nkv, hd, cr, sr))
        assert np.array_equal(f16_bits(kp[t]), e)


def test_kv_cache_write(cuda, orc):
    from nve_b200 import cuda_kernels as ck

    torch = cuda
    nkv, hd, max_seq, pos = 8, 128, 32, 17
    kc = torch.zeros((nkv, max_seq, hd), dtype=torch.float16, device="cuda")
    vc = torch.zeros_like(kc)
    kn = dev(orc.to_act16(orc.fill_normal(nkv * hd, 61, 1)), torch.float16).view(nkv, hd)
    vn = dev(orc.to_act16(orc.fill_normal(nkv * hd, 61, 2)), torch.float16).view(nkv, hd)
    d_pos = torch.tensor([pos], dtype=torch.int32, device="cuda")
    ck.kv_cache_write(kn, kc, vn, vc, d_pos.data_ptr(), nkv, hd, max_seq)
    assert torch.equal(kc[:, pos], kn) and torch.equal(vc[:, pos], vn)
    assert torch.count_nonzero(kc) == torch.count_nonzero(kn)
    # an out-of-range position is skipped, never written out of bounds
    d_pos.fill_(max_seq)
    before = kc.clone()
    ck.kv_cache_write(kn, kc, vn, vc, d_pos.data_ptr(), nkv, hd, max_seq)
    assert torch.equal(kc, before)


@pytest.mark.parametrize("nh,nkv,hd,seq", [(32, 8, 64, 1), (32, 8, 64, 77), (32, 8, 128, 1024), (64, 8, 128, 300),
                                           (4, 4, 256, 33), (2, 1, 512, 19), (8, 8, 32, 5)])
def test_flash_decode(cuda, orc, nh, nkv, hd, seq):
    from nve_b200 import cuda_kernels as ck

    torch = cuda
    q16 = orc.to_act16(orc.fill_normal(nh * hd, 71, 1))
    k16 = orc.to_act16(orc.fill_normal(nkv * seq * hd, 71, 2))
    v16 = orc.to_act16(orc.fill_normal(nkv * seq * hd, 71, 3))
    scale = hd ** -0.5
    ref = orc.attn_decode(orc.from_act16(q16).reshape(nh, hd), orc.from_act16(k16).reshape(nkv, seq, hd),
                          orc.from_act16(v16).reshape(nkv, seq, hd), seq, scale)
    q = dev(q16, torch.float16).view(nh, hd)
    kc = dev(k16, torch.float16).view(nkv, seq, hd)
    vc = dev(v16, torch.float16).view(nkv, seq, hd)
    out = ck.flash_decode_f16(q, kc, vc, nh, nkv, scale)
    assert rel_rms_err(out.float().cpu().numpy(), ref) < 5e-3
    # device-length form over a larger static cache
    max_seq = seq + 13
    kbig = torch.zeros((nkv, max_seq, hd), dtype=torch.float16, device="cuda")
    vbig = torch.zeros_like(kbig)
    kbig[:, :seq] = kc
    vbig[:, :seq] = vc
    kbig[:, seq:] = 100.0  # must not be read
    out2 = torch.empty_like(out)
    d_len = torch.tensor([seq], dtype=torch.int32, device="cuda")
    ck.flash_decode_dyn_into(q, kbig, vbig, out2, nh, nkv, d_len.data_ptr(), hd, scale, max_seq)
    assert torch.equal(out2, out)


@pytest.mark.parametrize("nh,nkv,hd,pos", [(32, 8, 64, 0), (32, 8, 128, 100), (64, 8, 128, 1023), (8, 8, 64, 5), (6, 2, 128, 40),
                                           (32, 8, 128, 1023), (32, 8, 128, 127), (32, 8, 128, 128), (16, 8, 64, 129),
                                           (8, 2, 128, 7), (4, 4, 128, 1000), (32, 8, 128, 15), (32, 8, 128, 16),
                                           (64, 8, 64, 50), (16, 2, 128, 300), (8, 1, 64, 1),
                                           # long contexts: several 16-position tiles per warp of the tensor-core kernel
                                           (32, 8, 128, 4000), (16, 2, 64, 2500), (16, 2, 128, 3071)])
def test_fused_attention_equals_separate_launches(cuda, orc, nh, nkv, hd, pos):
    """RoPE + KV write + attention + quantise in one launch == the four separate launches, bit for bit, with either
    attention kernel (the un-fused entry points run the same kernel as the fused one); the tensor-core and the
    CUDA-core kernel agree with each other within rounding."""
    from nve_b200 import cuda_kernels as ck

    torch = cuda
    max_seq = 1024 if pos < 1024 else 4096
    c16, s16, dc, ds = _rope_tables(orc, torch, hd, max_seq)
    q = dev(orc.to_act16(orc.fill_normal(nh * hd, 75, 1)), torch.float16).view(nh, hd)
    k = dev(orc.to_act16(orc.fill_normal(nkv * hd, 75, 2)), torch.float16).view(nkv, hd)
    v = dev(orc.to_act16(orc.fill_normal(nkv * hd, 75, 3)), torch.float16).view(nkv, hd)
    kc = dev(orc.to_act16(orc.fill_normal(nkv * max_seq * hd, 75, 4)), torch.float16).view(nkv, max_seq, hd)
    vc = dev(orc.to_act16(orc.fill_normal(nkv * max_seq * hd, 75, 5)), torch.float16).view(nkv, max_seq, hd)
    d_pos = torch.tensor([pos], dtype=torch.int32, device="cuda")
    d_len = torch.tensor([pos + 1], dtype=torch.int32, device="cuda")
    scale = hd ** -0.5
    outs = {}
    for cuda_core in (True, False):
        with ck.attn_decode_kernel(cuda_core=cuda_core):
            # separate launches (the reference's sequence)
            q1, k1, kc1, vc1 = q.clone(), k.clone(), kc.clone(), vc.clone()
            ck.rope_decode_dyn_inplace(q1, k1, dc, ds, nh, nkv, hd, d_pos.data_ptr())
            ck.kv_cache_write(k1, kc1, v, vc1, d_pos.data_ptr(), nkv, hd, max_seq)
            out1 = torch.empty((nh, hd), dtype=torch.float16, device="cuda")
            ck.flash_decode_dyn_into(q1, kc1, vc1, out1, nh, nkv, d_len.data_ptr(), hd, scale, max_seq)
            xq1, xs1 = ck.quantize_f16_q8(out1)
            # one launch
            kc2, vc2 = kc.clone(), vc.clone()
            out2 = torch.empty_like(out1)
            xq2 = torch.empty(nh * hd, dtype=torch.int8, device="cuda")
            xs2 = torch.empty(nh * hd // 32, dtype=torch.float32, device="cuda")
            ck.attn_decode_fused(q, k, v, kc2, vc2, dc, ds, d_pos.data_ptr(), d_len.data_ptr(), out2, nh, nkv, hd, max_seq, scale,
                                 out_q=xq2, out_scales=xs2)
            out4 = torch.empty_like(out1)  # without the quantised output
            ck.attn_decode_fused(q, k, v, kc.clone(), vc.clone(), dc, ds, d_pos.data_ptr(), d_len.data_ptr(), out4, nh, nkv, hd,
                                 max_seq, scale)
        assert torch.equal(out2, out1) and torch.equal(kc2, kc1) and torch.equal(vc2, vc1), f"cuda_core={cuda_core}"
        assert torch.equal(xq2, xq1) and torch.equal(xs2, xs1)
        assert torch.equal(out4, out2)
        outs[cuda_core] = out2
    # the two kernels agree within rounding (f16 probabilities, another summation order)
    assert (outs[False].float() - outs[True].float()).abs().max().item() < 5e-3 * max(1.0, outs[True].float().abs().max().item())
    # and against the oracle
    ref = orc.attn_decode(orc.from_act16(f16_bits(q1)).reshape(nh, hd), kc1.float().cpu().numpy(), vc1.float().cpu().numpy(),
                          pos + 1, scale)
    assert rel_rms_err(out2.float().cpu().numpy(), ref) < 5e-3


@pytest.mark.parametrize("route", ["w4a8", "w4a16"])
def test_rmsnorm_prologue_gemv_equals_separate_launches(cuda, orc, route):
    from nve_b200 import cuda_kernels as ck

    torch = cuda
    K = 4096
    mats = []
    for i, N in enumerate((1024, 256, 256)):
        W = orc.fill_normal(N * K, 77, i, scale=0.02).reshape(N, K)
        nib, sc = orc.extract_for_gpu(orc.quantize_q4(W))
        mats.append((dev(nib), dev(sc), N))
    h = dev(orc.to_act16(orc.fill_normal(K, 77, 9) * 3.0), torch.float16).view(1, -1)
    w = dev(orc.to_act16(1.0 + 0.1 * orc.fill_normal(K, 77, 10)), torch.float16)
    if route == "w4a8":
        xq, xs, _ = ck.rmsnorm_quantize_q8(h, w, 1e-5)
        sep = ck.matvec_w4a8_multi(xq, xs, mats, K)
        fused = ck.rmsnorm_matvec_w4a8_multi(h, w, 1e-5, mats, K)
    else:
        normed = ck.fused_rms_norm(h, w, 1e-5)
        sep = ck.matvec_w4a16_multi(normed, None, mats, K)
        fused = ck.rmsnorm_matvec_w4a16_multi(h, w, 1e-5, None, mats, K)
    for a, b in zip(sep, fused):
        assert torch.equal(a, b)


# ------------------------------------------------------------------ decode layer and graph
def _make_state(torch, orc, hidden, ffn, nh, nkv, hd, layers, max_seq, seed, fused):
    from nve_b200 import cuda_kernels as ck
    from nve_b200.gpu_layer import GpuInferenceState, GpuKvCache, GpuLayerWeights, GpuW4, RoutingConfig

    def w4(n, k, sid):
        W = ck.fill_normal(n * k, seed, sid, scale=0.02).view(n, k)
        nib, sc = ck.q4_quantize(W)
        return GpuW4(nib, sc, None, n, k)

    lw = []
    for li in range(layers):
        b = 100 * li
        ones = torch.ones(hidden, dtype=torch.float16, device="cuda")
        lw.append(GpuLayerWeights(w4(nh * hd, hidden, b + 1), w4(nkv * hd, hidden, b + 2), w4(nkv * hd, hidden, b + 3),
                                  w4(hidden, nh * hd, b + 4), w4(ffn, hidden, b + 5), w4(ffn, hidden, b + 6),
                                  w4(hidden, ffn, b + 7), ones, ones.clone()))
    cos, sin = orc.rope_tables_f32(hd, max_seq, 10000.0)
    kv = GpuKvCache(layers, nkv, max_seq, hd, "cuda")
    return GpuInferenceState(lw, kv, nh, nkv, hd, 1e-5, dev(orc.to_act16(cos), torch.float16),
                             dev(orc.to_act16(sin), torch.float16), RoutingConfig(False, 0.7), fused)


def _oracle_layer(orc, h16, w, kc_f32, vc_f32, pos, nh, nkv, hd, cos16, sin16, use_w4a8):
    """One decode layer on the host with the oracle pieces, mirroring src/gpu_layer.rs:1027-1083 (16-bit
    activations between kernels, as the device path has them)."""
    def cpu(t):
        return t.cpu().numpy()

    def gemv(x16, p):
        nib, sc = cpu(p.nibbles), cpu(p.scales)
        if use_w4a8:
            xq, xs = orc.quantize_q8(x16)
            return orc.to_act16(orc.w4a8_matvec_f64(xq, xs, nib, sc).astype(np.float32))
        return orc.to_act16(orc.w4a16_matvec_f64(orc.from_act16(x16), nib, sc).astype(np.float32))

    ones = orc.to_act16(np.ones(h16.size, np.float32))
    n1 = orc.rms_norm_16(h16, ones, 1e-5)
    q = orc.from_act16(gemv(n1, w.q_proj))
    k = orc.from_act16(gemv(n1, w.k_proj))
    v16 = gemv(n1, w.v_proj)
    cr, sr = orc.from_act16(cos16[pos]), orc.from_act16(sin16[pos])
    q = orc.from_act16(orc.to_act16(orc.rope_apply(q, nh, hd, cr, sr)))
    k = orc.from_act16(orc.to_act16(orc.rope_apply(k, nkv, hd, cr, sr)))
    kc_f32[:, pos] = k.reshape(nkv, hd)
    vc_f32[:, pos] = orc.from_act16(v16).reshape(nkv, hd)
    attn = orc.to_act16(orc.attn_decode(q.reshape(nh, hd), kc_f32, vc_f32, pos + 1, hd ** -0.5).reshape(-1))
    o = gemv(attn, w.o_proj)
    h1 = orc.to_act16(orc.from_act16(h16) + orc.from_act16(o))
    n2 = orc.rms_norm_16(h1, ones, 1e-5)
    g, u = gemv(n2, w.gate_proj), gemv(n2, w.up_proj)
    mid = orc.silu_mul_16(g, u)
    d = gemv(mid, w.down_proj)
    return orc.to_act16(orc.from_act16(h1) + orc.from_act16(d))


@pytest.mark.parametrize("use_w4a8", [True, False])
@pytest.mark.parametrize("cuda_core_attention", [True, False])
def test_decode_layer_fused_equals_reference_sequence_and_oracle(cuda, orc, use_w4a8, cuda_core_attention):
    """The fused schedule against the reference's kernel sequence: bit for bit with either attention kernel; both
    within tolerance of a host oracle layer."""
    from nve_b200 import cuda_kernels as ck
    from nve_b200.gpu_layer import gpu_layer_forward_decode

    torch = cuda
    hidden, ffn, nh, nkv, hd, max_seq = 512, 1024, 8, 2, 64, 16
    importance = 0.0 if use_w4a8 else 1.0
    states = [_make_state(torch, orc, hidden, ffn, nh, nkv, hd, 1, max_seq, 81, fused) for fused in (True, False)]
    h16 = orc.to_act16(orc.fill_normal(hidden, 82, 1))
    cos, sin = orc.rope_tables_f32(hd, max_seq, 10000.0)
    cos16, sin16 = orc.to_act16(cos), orc.to_act16(sin)
    kc = np.zeros((nkv, max_seq, hd), np.float32)
    vc = np.zeros_like(kc)
    hs = [dev(h16, torch.float16).view(1, -1) for _ in states]
    h_or = h16
    for pos in range(3):
        with ck.attn_decode_kernel(cuda_core=cuda_core_attention):
            outs = [gpu_layer_forward_decode(h, 0, st, pos, False, importance) for h, st in zip(hs, states)]
        assert torch.equal(outs[0], outs[1])  # fused schedule == the reference's kernel sequence, bit for bit
        h_or = _oracle_layer(orc, h_or, states[0].layer_weights[0], kc, vc, pos, nh, nkv, hd, cos16, sin16, use_w4a8)
        assert rel_rms_err(outs[0].float().cpu().numpy(), orc.from_act16(h_or)) < TOL
        hs = outs


def test_graph_replay_equals_eager_mixed_routing(cuda, orc):
    from nve_b200 import cuda_kernels as ck
    from nve_b200.decode_graph import StaticDecodeGraph
    from nve_b200.gpu_layer import RoutingConfig, gpu_layer_forward_decode

    torch = cuda
    hidden, ffn, nh, nkv, hd, layers, max_seq = 512, 1024, 8, 2, 64, 4, 16
    imp = [0.1, 0.9, 0.4, 1.0]  # threshold 0.7: layers 0 and 2 run W4A8, 1 and 3 run W4A16
    st_e = _make_state(torch, orc, hidden, ffn, nh, nkv, hd, layers, max_seq, 91, True)
    st_g = _make_state(torch, orc, hidden, ffn, nh, nkv, hd, layers, max_seq, 91, True)
    graph = StaticDecodeGraph(st_g, hidden, ffn, imp)
    assert graph.routes == [True, False, True, False]
    graph.capture()
    assert graph.launches_per_replay == 6 * layers
    try:
        for pos in range(4):
            h_in = dev(orc.to_act16(orc.fill_normal(hidden, 92, pos)), torch.float16).view(1, -1)
            h = h_in
            for li in range(layers):
                h = gpu_layer_forward_decode(h, li, st_e, pos, False, imp[li])
            out = graph.replay(h_in, pos)
            torch.cuda.synchronize()
            assert torch.equal(out, h)
        for li in range(layers):
            assert torch.equal(st_e.kv_cache.k[li], st_g.kv_cache.k[li])
    finally:
        graph.destroy()
    assert not ck.graph_ready()


# ------------------------------------------------------------------ five launches per layer
@pytest.mark.parametrize("route", ["w4a8", "w4a16"])
@pytest.mark.parametrize("K,F", [(4096, 1024), (2048, 512), (1024, 264), (512, 96)])
def test_gateup_silu_epilogue_equals_gemv_plus_silu(cuda, orc, route, K, F):
    """RMSNorm + gate/up GEMV + SiLU*up in one launch == RMSNorm-fused gate/up GEMV followed by the SiLU*up kernel, bit
    for bit (2, 4 and 8 rows per item; F = 264 and 96 leave ragged last tiles)."""
    from nve_b200 import cuda_kernels as ck

    torch = cuda
    mats = []
    for i in range(2):
        W = orc.fill_normal(F * K, 771, i, scale=0.02).reshape(F, K)
        nib, sc = orc.extract_for_gpu(orc.quantize_q4(W))
        mats.append((dev(nib), dev(sc), F))
    h = dev(orc.to_act16(orc.fill_normal(K, 771, 9) * 3.0), torch.float16).view(1, -1)
    w = dev(orc.to_act16(1.0 + 0.1 * orc.fill_normal(K, 771, 10)), torch.float16)
    if route == "w4a8":
        gate, up = ck.rmsnorm_matvec_w4a8_multi(h, w, 1e-5, mats, K)
    else:
        gate, up = ck.rmsnorm_matvec_w4a16_multi(h, w, 1e-5, None, mats, K)
    ck.silu_mul_inplace(gate, up)
    mid = ck.rmsnorm_gateup_silu(h, w, 1e-5, None, mats[0], mats[1], K, route == "w4a8")
    assert torch.equal(mid, gate)


@pytest.mark.parametrize("route", ["w4a8", "w4a16"])
@pytest.mark.parametrize("K,F", [(4096, 14336), (2048, 512), (1024, 288), (512, 96)])
def test_gateup_silu_group_conversion_equals_activation_kernels(cuda, orc, route, K, F):
    """The quantising form of the fused gate/up launch leaves, besides mid, exactly what the stand-alone SiLU*up +
    quantise kernels leave for the down projection (int8 codes / 16-bit fixed-point planes + scales), on three launches
    in a row with different inputs over the same group counters (stale or double conversions would show)."""
    from nve_b200 import cuda_kernels as ck

    torch = cuda
    mats = []
    for i in range(2):
        W = orc.fill_normal(F * K, 775, i, scale=0.02).reshape(F, K)
        nib, sc = orc.extract_for_gpu(orc.quantize_q4(W))
        mats.append((dev(nib), dev(sc), F))
    w = dev(orc.to_act16(1.0 + 0.1 * orc.fill_normal(K, 775, 10)), torch.float16)
    awq = dev((1.0 + 0.25 * np.abs(orc.fill_normal(F, 775, 11))).astype(np.float32)) if route == "w4a16" else None
    cnt = torch.zeros(F // 32, dtype=torch.int32, device="cuda")
    xq = torch.full((F,), 99, dtype=torch.int8, device="cuda")
    xlo = torch.full((F,), 99, dtype=torch.uint8, device="cuda")
    xs = torch.full((F // 32,), -1.0, dtype=torch.float32, device="cuda")
    for call in range(3):
        h = dev(orc.to_act16(orc.fill_normal(K, 775, 20 + call) * (3.0 + call)), torch.float16).view(1, -1)
        if route == "w4a8":
            gate, up = ck.rmsnorm_matvec_w4a8_multi(h, w, 1e-5, mats, K)
            want_q = torch.empty((F,), dtype=torch.int8, device="cuda")
            want_s = torch.empty((F // 32,), dtype=torch.float32, device="cuda")
            want_mid = ck.silu_mul_quantize_q8(gate, up, want_mid=True, xq=want_q, scales=want_s)[2]
            mid = ck.rmsnorm_gateup_silu(h, w, 1e-5, None, mats[0], mats[1], K, True,
                                         quant={"xq": xq, "xs": xs, "counters": cnt})
            torch.cuda.synchronize()
            assert torch.equal(xq, want_q) and torch.equal(xs, want_s), f"call {call}"
        else:
            gate, up = ck.rmsnorm_matvec_w4a16_multi(h, w, 1e-5, None, mats, K)
            want_lo = torch.empty((F,), dtype=torch.uint8, device="cuda")
            want_hi = torch.empty((F,), dtype=torch.int8, device="cuda")
            want_s = torch.empty((F // 32,), dtype=torch.float32, device="cuda")
            want_mid = ck.silu_mul_x16(gate, up, awq, want_mid=True, x_lo=want_lo, x_hi=want_hi, scales=want_s)[3]
            mid = ck.rmsnorm_gateup_silu(h, w, 1e-5, None, mats[0], mats[1], K, False,
                                         quant={"xlo": xlo, "xhi": xq, "xs": xs, "counters": cnt, "down_awq": awq})
            torch.cuda.synchronize()
            assert torch.equal(xlo, want_lo) and torch.equal(xq, want_hi) and torch.equal(xs, want_s), f"call {call}"
        assert int(cnt.min()) == 32 * (call + 1) and int(cnt.max()) == 32 * (call + 1)
        assert torch.equal(mid, want_mid)


def test_quantizing_prologue_equals_quantiser_plus_gemv(cuda, orc):
    from nve_b200 import cuda_kernels as ck

    torch = cuda
    N, K = 512, 14336
    W = orc.fill_normal(N * K, 781, 1, scale=0.02).reshape(N, K)
    nib, sc = orc.extract_for_gpu(orc.quantize_q4(W))
    mats = [(dev(nib), dev(sc), N)]
    x = dev(orc.to_act16(orc.fill_normal(K, 781, 2)), torch.float16).view(1, -1)
    res = dev(orc.to_act16(orc.fill_normal(N, 781, 3)), torch.float16).view(1, -1)
    xq, xs = ck.quantize_f16_q8(x)
    want = ck.matvec_w4a8_multi(xq, xs, mats, K, residuals=[res])[0]
    got = ck.quantize_matvec_w4a8_multi(x, None, mats, K, residuals=[res])[0]
    assert torch.equal(got, want)


def test_five_launch_graph_equals_six_launch_graph(cuda, orc):
    from nve_b200.decode_graph import StaticDecodeGraph

    torch = cuda
    hidden, ffn, nh, nkv, hd, layers, max_seq = 2048, 8192, 32, 8, 64, 4, 16
    imp = [0.1, 0.9, 0.4, 1.0]
    outs = []
    # six launches; five with the conversion at the tail of the gate/up launch; five with it in the down prologue
    for fuse, in_prologue in ((False, False), (True, False), (True, True)):
        st = _make_state(torch, orc, hidden, ffn, nh, nkv, hd, layers, max_seq, 791, True)
        st.fuse_silu = fuse
        st.convert_in_down_prologue = in_prologue
        graph = StaticDecodeGraph(st, hidden, ffn, imp)
        graph.capture()
        assert graph.launches_per_replay == (5 if fuse else 6) * layers
        try:
            res = []
            for pos in range(3):
                h_in = dev(orc.to_act16(orc.fill_normal(hidden, 792, pos)), torch.float16).view(1, -1)
                res.append(graph.replay(h_in, pos))
                torch.cuda.synchronize()
            outs.append(res)
        finally:
            graph.destroy()
    for other in outs[1:]:
        for a, b in zip(outs[0], other):
            assert torch.equal(a, b)


# ------------------------------------------------------------------ prefill: a block of positions through one layer
def test_rms_norm_rows_and_kv_rows_write(cuda, orc):
    from nve_b200 import cuda_kernels as ck

    torch = cuda
    S, n = 7, 2048
    x = dev(orc.to_act16(orc.fill_normal(S * n, 811, 1) * 2.0), torch.float16).view(S, n)
    w = dev(orc.to_act16(1.0 + 0.1 * orc.fill_normal(n, 811, 2)), torch.float16)
    got = ck.rms_norm_rows(x, w, 1e-5)
    for r in range(S):
        assert torch.equal(got[r], ck.rms_norm(x[r].contiguous(), w, 1e-5))
    nkv, hd, max_seq, start = 4, 64, 32, 9
    k_new = dev(orc.to_act16(orc.fill_normal(S * nkv * hd, 811, 3)), torch.float16).view(S, nkv, hd)
    v_new = dev(orc.to_act16(orc.fill_normal(S * nkv * hd, 811, 4)), torch.float16).view(S, nkv, hd)
    kc = torch.zeros((nkv, max_seq, hd), dtype=torch.float16, device="cuda")
    vc = torch.zeros_like(kc)
    ck.kv_cache_write_rows(k_new, kc, v_new, vc, start, nkv, hd, max_seq)
    want_k, want_v = torch.zeros_like(kc), torch.zeros_like(vc)
    want_k[:, start:start + S] = k_new.transpose(0, 1)
    want_v[:, start:start + S] = v_new.transpose(0, 1)
    assert torch.equal(kc, want_k) and torch.equal(vc, want_v)


@pytest.mark.parametrize("nh,nkv,hd", [(32, 8, 128), (8, 8, 64), (12, 4, 64)])
def test_attn_prefill_causal_rows_equal_decode_calls(cuda, orc, nh, nkv, hd):
    """Every row of the one-launch causal attention equals a flash-decode call of that row's length, bit for bit
    (blocks of fewer than 64 (row, KV head) pairs, which run the decode kernel)."""
    from nve_b200 import cuda_kernels as ck

    torch = cuda
    S, start, max_seq = 7, 37, 64
    q = dev(orc.to_act16(orc.fill_normal(S * nh * hd, 821, 1)), torch.float16).view(S, nh * hd)
    kc = dev(orc.to_act16(orc.fill_normal(nkv * max_seq * hd, 821, 2)), torch.float16).view(nkv, max_seq, hd)
    vc = dev(orc.to_act16(orc.fill_normal(nkv * max_seq * hd, 821, 3)), torch.float16).view(nkv, max_seq, hd)
    got = ck.attn_prefill_causal(q, kc, vc, start, nh, nkv, hd, max_seq, hd ** -0.5)
    d_len = torch.zeros(1, dtype=torch.int32, device="cuda")
    for r in range(S):
        d_len.fill_(start + r + 1)
        want = torch.empty((nh * hd,), dtype=torch.float16, device="cuda")
        ck.flash_decode_dyn_into(q[r].contiguous(), kc, vc, want, nh, nkv, d_len.data_ptr(), hd, hd ** -0.5, max_seq)
        torch.cuda.synchronize()
        assert torch.equal(got[r], want), f"row {r}"


@pytest.mark.parametrize("nh,nkv,hd,S,start,max_seq", [(32, 8, 128, 40, 21, 64), (8, 8, 64, 130, 0, 160), (12, 4, 64, 33, 300, 333),
                                                       (8, 1, 128, 64, 5, 80)])
def test_attn_prefill_causal_large_blocks_match_decode_calls(cuda, orc, nh, nkv, hd, S, start, max_seq):
    """Blocks of 64 or more (row, KV head) pairs run the tensor-core kernel: every row within rounding of the
    flash-decode call of that row's length (f16 probabilities and a different summation order)."""
    from nve_b200 import cuda_kernels as ck

    torch = cuda
    q = dev(orc.to_act16(orc.fill_normal(S * nh * hd, 841, 1)), torch.float16).view(S, nh * hd)
    kc = dev(orc.to_act16(orc.fill_normal(nkv * max_seq * hd, 841, 2)), torch.float16).view(nkv, max_seq, hd)
    vc = dev(orc.to_act16(orc.fill_normal(nkv * max_seq * hd, 841, 3)), torch.float16).view(nkv, max_seq, hd)
    got = ck.attn_prefill_causal(q, kc, vc, start, nh, nkv, hd, max_seq, hd ** -0.5)
    d_len = torch.zeros(1, dtype=torch.int32, device="cuda")
    want = torch.empty((S, nh * hd), dtype=torch.float16, device="cuda")
    for r in range(S):
        d_len.fill_(start + r + 1)
        ck.flash_decode_dyn_into(q[r].contiguous(), kc, vc, want[r], nh, nkv, d_len.data_ptr(), hd, hd ** -0.5, max_seq)
        torch.cuda.synchronize()
    err = (got.float() - want.float()).abs().max().item()
    assert err < 5e-3 * max(1.0, want.float().abs().max().item()), err


def test_prefill_layers_match_sequential_decode(cuda, orc):
    """gpu_layer_forward_prefill on a block of S positions against S sequential decode steps through the same two
    layers (16-bit route on every layer, as in the reference's prefill): hidden states within the tolerance that
    separates the f16-dequantised tensor-core GEMM from the integer GEMV, K/V caches likewise (the reference tests
    prefill-vs-sequential agreement in tests/e2e.rs:440-479)."""
    from nve_b200.gpu_layer import gpu_layer_forward_decode, gpu_layer_forward_prefill

    torch = cuda
    hidden, ffn, nh, nkv, hd, layers, max_seq, S, start = 1024, 2816, 16, 4, 64, 2, 32, 6, 3
    st_d = _make_state(torch, orc, hidden, ffn, nh, nkv, hd, layers, max_seq, 831, True)
    st_p = _make_state(torch, orc, hidden, ffn, nh, nkv, hd, layers, max_seq, 831, True)
    st_d.routing.no_w4a8 = True
    # both caches start with the same `start` earlier positions
    for li in range(layers):
        for t, sid in ((st_d.kv_cache.k, 1), (st_d.kv_cache.v, 2)):
            t[li][:, :start] = dev(orc.to_act16(orc.fill_normal(nkv * start * hd, 832, 10 * li + sid)), torch.float16).view(
                nkv, start, hd)
        st_p.kv_cache.k[li].copy_(st_d.kv_cache.k[li])
        st_p.kv_cache.v[li].copy_(st_d.kv_cache.v[li])
    x = dev(orc.to_act16(orc.fill_normal(S * hidden, 833, 1)), torch.float16).view(S, hidden)
    # sequential decode
    seq_out = []
    for s in range(S):
        h = x[s:s + 1].contiguous()
        for li in range(layers):
            h = gpu_layer_forward_decode(h, li, st_d, start + s, False, 1.0)
        seq_out.append(h)
    seq_out = torch.cat(seq_out)
    # block prefill
    hp = x
    for li in range(layers):
        hp = gpu_layer_forward_prefill(hp, li, st_p, start)
    torch.cuda.synchronize()
    assert rel_rms_err(hp.float().cpu().numpy(), seq_out.float().cpu().numpy()) < 5e-3
    for li in range(layers):
        for a, b in ((st_p.kv_cache.k[li], st_d.kv_cache.k[li]), (st_p.kv_cache.v[li], st_d.kv_cache.v[li])):
            assert rel_rms_err(a[:, :start + S].float().cpu().numpy(), b[:, :start + S].float().cpu().numpy()) < 5e-3


# ------------------------------------------------------------------ batched decode: several sequences per step
@pytest.mark.parametrize("cuda_core", [False, True])
def test_attn_decode_fused_batch_rows_equal_single_calls(cuda, orc, cuda_core):
    """Every row of the batched fused attention (RoPE + K/V write + attention) equals the single-sequence launch on
    that sequence's cache, position and length, bit for bit -- output and the cache row written -- with either
    clustered kernel (few sequences run the kernel a single sequence would)."""
    from nve_b200 import cuda_kernels as ck

    torch = cuda
    B, nh, nkv, hd, max_seq = 5, 32, 8, 128, 40
    pos = [0, 7, 39, 18, 3]
    q = dev(orc.to_act16(orc.fill_normal(B * nh * hd, 851, 1)), torch.float16).view(B, nh * hd)
    k = dev(orc.to_act16(orc.fill_normal(B * nkv * hd, 851, 2)), torch.float16).view(B, nkv * hd)
    v = dev(orc.to_act16(orc.fill_normal(B * nkv * hd, 851, 3)), torch.float16).view(B, nkv * hd)
    kc = dev(orc.to_act16(orc.fill_normal(B * nkv * max_seq * hd, 851, 4)), torch.float16).view(B, nkv, max_seq, hd)
    vc = dev(orc.to_act16(orc.fill_normal(B * nkv * max_seq * hd, 851, 5)), torch.float16).view(B, nkv, max_seq, hd)
    cos, sin = orc.rope_tables_f32(hd, max_seq, 10000.0)
    cos, sin = dev(orc.to_act16(cos), torch.float16), dev(orc.to_act16(sin), torch.float16)
    d_pos = torch.tensor(pos, dtype=torch.int32, device="cuda")
    d_len = d_pos + 1
    kc_b, vc_b = kc.clone(), vc.clone()
    with ck.attn_decode_kernel(cuda_core=cuda_core):
        got = ck.attn_decode_fused_batch(q, k, v, kc_b, vc_b, cos, sin, d_pos, d_len, nh, nkv, hd, max_seq, hd ** -0.5)
    for b in range(B):
        kc_s, vc_s = kc[b].clone(), vc[b].clone()
        want = torch.empty((nh, hd), dtype=torch.float16, device="cuda")
        with ck.attn_decode_kernel(cuda_core=cuda_core):
            ck.attn_decode_fused(q[b].view(nh, hd).contiguous(), k[b].view(nkv, hd).contiguous(), v[b].view(nkv, hd).contiguous(),
                                 kc_s, vc_s, cos, sin, d_pos[b:b + 1].data_ptr(), d_len[b:b + 1].data_ptr(), want, nh, nkv, hd,
                                 max_seq, hd ** -0.5)
        torch.cuda.synchronize()
        assert torch.equal(got[b].view(nh, hd), want), f"sequence {b}"
        assert torch.equal(kc_b[b], kc_s) and torch.equal(vc_b[b], vc_s), f"cache of sequence {b}"


def test_batched_decode_layers_match_single_sequence_decode(cuda, orc):
    """gpu_layer_forward_decode_batch on B sequences at different positions against B single-sequence decode steps
    (16-bit route) through the same two layers."""
    from nve_b200 import cuda_kernels as ck
    from nve_b200.gpu_layer import BatchedKvCache, gpu_layer_forward_decode, gpu_layer_forward_decode_batch

    torch = cuda
    hidden, ffn, nh, nkv, hd, layers, max_seq, B = 1024, 2816, 16, 4, 64, 2, 32, 4
    pos = [5, 0, 31, 12]
    st = _make_state(torch, orc, hidden, ffn, nh, nkv, hd, layers, max_seq, 861, True)
    st.routing.no_w4a8 = True
    kvb = BatchedKvCache.zeros(layers, B, nkv, max_seq, hd)
    for li in range(layers):
        kvb.k[li].copy_(dev(orc.to_act16(orc.fill_normal(B * nkv * max_seq * hd, 862, 2 * li)), torch.float16).view(B, nkv, max_seq, hd))
        kvb.v[li].copy_(dev(orc.to_act16(orc.fill_normal(B * nkv * max_seq * hd, 862, 2 * li + 1)), torch.float16).view(B, nkv, max_seq, hd))
    x = dev(orc.to_act16(orc.fill_normal(B * hidden, 863, 1)), torch.float16).view(B, hidden)
    # single-sequence reference: one state per sequence, its cache = that sequence's slice
    want = []
    caches = []
    for b in range(B):
        for li in range(layers):
            st.kv_cache.k[li].copy_(kvb.k[li][b])
            st.kv_cache.v[li].copy_(kvb.v[li][b])
        h = x[b:b + 1].contiguous()
        for li in range(layers):
            h = gpu_layer_forward_decode(h, li, st, pos[b], False, 1.0)
        want.append(h)
        caches.append([(st.kv_cache.k[li].clone(), st.kv_cache.v[li].clone()) for li in range(layers)])
    want = torch.cat(want)
    d_pos = torch.tensor(pos, dtype=torch.int32, device="cuda")
    d_len = d_pos + 1
    # the allocation-free form (pre-allocated scratch) on a copy of the caches gives the same bits as the allocating one
    from nve_b200.gpu_layer import BatchedDecodeScratch

    kvb2 = BatchedKvCache([t.clone() for t in kvb.k], [t.clone() for t in kvb.v], B, max_seq)
    scratch = BatchedDecodeScratch.make(st, B, hidden, ffn)
    hb2 = x
    for li in range(layers):
        hb2 = gpu_layer_forward_decode_batch(hb2, li, st, kvb2, d_pos, d_len, scratch)
    hb = x
    for li in range(layers):
        hb = gpu_layer_forward_decode_batch(hb, li, st, kvb, d_pos, d_len)
    torch.cuda.synchronize()
    assert torch.equal(hb, hb2)
    # the residual add at the end of a layer deferred into the next layer's first launch: same bits
    kvb3 = BatchedKvCache([t.clone() for t in kvb2.k], [t.clone() for t in kvb2.v], B, max_seq)
    hb3, res = x, None
    for li in range(layers):
        r = gpu_layer_forward_decode_batch(hb3, li, st, kvb3, d_pos, d_len, scratch, residual=res, defer_add=li < layers - 1)
        hb3, res = r if li < layers - 1 else (r, None)
    torch.cuda.synchronize()
    assert torch.equal(hb3, hb)
    # the fused add + RMSNorm launch against the two kernels
    xa = dev(orc.to_act16(orc.fill_normal(B * hidden, 861, 1)), torch.float16).view(B, hidden)
    da = dev(orc.to_act16(orc.fill_normal(B * hidden, 861, 2)), torch.float16).view(B, hidden)
    wn = dev(orc.to_act16(1.0 + 0.1 * orc.fill_normal(hidden, 861, 3)), torch.float16)
    x1, x2 = xa.clone(), xa.clone()
    n1 = ck.add_rms_norm_rows(x1, da, wn, 1e-5)
    ck.add_inplace_any(x2, da)
    n2 = ck.rms_norm_rows(x2, wn, 1e-5)
    assert torch.equal(x1, x2) and torch.equal(n1, n2)
    assert rel_rms_err(hb.float().cpu().numpy(), want.float().cpu().numpy()) < 5e-3
    for b in range(B):
        for li in range(layers):
            assert rel_rms_err(kvb.k[li][b].float().cpu().numpy(), caches[b][li][0].float().cpu().numpy()) < 5e-3
            assert rel_rms_err(kvb.v[li][b].float().cpu().numpy(), caches[b][li][1].float().cpu().numpy()) < 5e-3


@pytest.mark.parametrize("B,nh,nkv,hd", [(24, 32, 8, 128), (20, 16, 16, 64), (24, 64, 8, 64), (80, 4, 2, 128),
                                         (24, 24, 8, 128)])
def test_attn_decode_fused_batch_large_batch_forms(cuda, orc, B, nh, nkv, hd):
    """With enough sequences the batched attention runs one CTA per (sequence, KV head) over all positions on the
    tensor cores (group sizes 1, 2, 4, 8; the probabilities are rounded to f16 for the p.V product; other group sizes
    stay on the clustered kernel): rows agree with single-sequence launches within that rounding, and the cache rows
    written are bit-identical."""
    from nve_b200 import cuda_kernels as ck

    torch = cuda
    max_seq = 96
    assert B * nkv >= 64  # the dispatch threshold of nve_b200_attn_decode_fused_batch
    pos = [(7 * b + 3) % max_seq for b in range(B)]
    pos[0], pos[1] = 0, max_seq - 1
    q = dev(orc.to_act16(orc.fill_normal(B * nh * hd, 871, 1)), torch.float16).view(B, nh * hd)
    k = dev(orc.to_act16(orc.fill_normal(B * nkv * hd, 871, 2)), torch.float16).view(B, nkv * hd)
    v = dev(orc.to_act16(orc.fill_normal(B * nkv * hd, 871, 3)), torch.float16).view(B, nkv * hd)
    kc = dev(orc.to_act16(orc.fill_normal(B * nkv * max_seq * hd, 871, 4)), torch.float16).view(B, nkv, max_seq, hd)
    vc = dev(orc.to_act16(orc.fill_normal(B * nkv * max_seq * hd, 871, 5)), torch.float16).view(B, nkv, max_seq, hd)
    cos, sin = orc.rope_tables_f32(hd, max_seq, 10000.0)
    cos, sin = dev(orc.to_act16(cos), torch.float16), dev(orc.to_act16(sin), torch.float16)
    d_pos = torch.tensor(pos, dtype=torch.int32, device="cuda")
    d_len = d_pos + 1
    kc_b, vc_b = kc.clone(), vc.clone()
    got = ck.attn_decode_fused_batch(q, k, v, kc_b, vc_b, cos, sin, d_pos, d_len, nh, nkv, hd, max_seq, hd ** -0.5)
    for b in range(B):
        kc_s, vc_s = kc[b].clone(), vc[b].clone()
        want = torch.empty((nh, hd), dtype=torch.float16, device="cuda")
        ck.attn_decode_fused(q[b].view(nh, hd).contiguous(), k[b].view(nkv, hd).contiguous(), v[b].view(nkv, hd).contiguous(),
                             kc_s, vc_s, cos, sin, d_pos[b:b + 1].data_ptr(), d_len[b:b + 1].data_ptr(), want, nh, nkv, hd,
                             max_seq, hd ** -0.5)
        torch.cuda.synchronize()
        assert rel_rms_err(got[b].float().cpu().numpy().reshape(-1), want.float().cpu().numpy().reshape(-1)) < 5e-3, f"sequence {b}"
        assert torch.equal(kc_b[b], kc_s) and torch.equal(vc_b[b], vc_s), f"cache of sequence {b}"
