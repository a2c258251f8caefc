"""CPU: the oracle against the committed golden vectors, the reference's own unit-test cases, hand-computed
known answers, and the independent numpy restatement."""
import hashlib

import numpy as np
import pytest

from oracle import np_oracle as npo


def same_bits(a, b):
    a, b = np.asarray(a), np.asarray(b)
    return a.shape == b.shape and a.dtype == b.dtype and a.tobytes() == b.tobytes()


# ------------------------------------------------------------------ golden vectors
def test_golden_weight_quantizer(orc, golden):
    blocks = orc.quantize_q4(golden["w_edge"])
    assert same_bits(blocks, golden["w_edge_blocks"])
    nib, sc = orc.extract_for_gpu(blocks)
    assert same_bits(nib, golden["w_edge_nibbles"]) and same_bits(sc, golden["w_edge_scales"])


@pytest.mark.parametrize("tag,bf", [("f16", False), ("bf16", True)])
def test_golden_activation_quantizer(orc, golden, tag, bf):
    xq, xs = orc.quantize_q8(golden[f"act_{tag}"], bf)
    assert same_bits(xq, golden[f"act_{tag}_q"]) and same_bits(xs, golden[f"act_{tag}_s"])


def test_golden_gemv(orc, golden):
    g = golden
    xf = orc.from_act16(g["g_x16"])
    assert same_bits(orc.w4a8_idot(g["g_xq"], g["g_nibbles"]), g["g_idot"])
    assert same_bits(orc.w4a8_matvec_f64(g["g_xq"], g["g_xs"], g["g_nibbles"], g["g_scales"]), g["g_y_w4a8_f64"])
    assert same_bits(orc.w4a8_matvec_b200(g["g_xq"], g["g_xs"], g["g_nibbles"], g["g_scales"]), g["g_y_w4a8_b200"])
    assert same_bits(orc.w4a8_matvec_reforder(g["g_xq"], g["g_xs"], g["g_nibbles"], g["g_scales"]), g["g_y_w4a8_reforder"])
    assert same_bits(orc.q4_matvec(g["g_blocks"], xf, order="scalar"), g["g_y_cpu_scalar"])
    assert same_bits(orc.q4_matvec(g["g_blocks"], xf, order="avx2"), g["g_y_cpu_avx2"])
    assert same_bits(orc.w4a16_matvec_b200(g["g_x16"], g["g_nibbles"], g["g_scales"]), g["g_y_w4a16_b200"])
    assert same_bits(orc.w4a16_matvec_b200(g["g_x16"], g["g_awq_nibbles"], g["g_awq_scales"], g["g_awq_inv"]), g["g_y_awq_b200"])
    assert same_bits(orc.q4_matvec(orc.quantize_q4(g["g_w"], g["g_awq"]), xf, g["g_awq_inv"]), g["g_y_awq_cpu_scalar"])


def test_golden_glue(orc, golden):
    assert same_bits(orc.rms_norm_16(golden["n_x16"], golden["n_w16"], 1e-5), golden["n_out16"])
    assert same_bits(orc.normalize_importance(golden["r_scores"]), golden["r_norm"])


def test_golden_config1_digest(orc, golden):
    """Measurement configuration 1 (8192 x 2048 W4A16 GEMV) regenerated from the seed: digests of weights and outputs."""
    seed = int(golden["seed"][0])
    W = orc.fill_normal(8192 * 2048, seed, 10, scale=0.02).reshape(8192, 2048)
    x16 = orc.to_act16(orc.fill_normal(2048, seed, 11))
    blocks = orc.quantize_q4(W)
    nib, sc = orc.extract_for_gpu(blocks)
    sha = lambda a: np.frombuffer(hashlib.sha256(a.tobytes()).digest(), np.uint8)
    assert same_bits(sha(nib), golden["c1_nibbles_sha"]) and same_bits(sha(sc), golden["c1_scales_sha"])
    y = orc.q4_matvec(blocks, orc.from_act16(x16))
    assert same_bits(sha(y), golden["c1_y_cpu_scalar_sha"]) and same_bits(y[:64], golden["c1_y_cpu_scalar_head"])
    yb = orc.w4a16_matvec_b200(x16, nib, sc)
    assert same_bits(sha(yb), golden["c1_y_b200_sha"])
    # the integer formulation the CUDA library uses stays far inside the stated tolerance of the CPU path
    assert np.max(np.abs(yb - y)) / golden["c1_y_rms"][0] < 1e-3


# ------------------------------------------------------------------ the reference's own unit tests, restated
def test_ref_quantize_block_q4_roundtrip(orc):
    """src/quantize.rs:2234-2252: values (i-16)*0.5, |orig - dequant| < 2.0."""
    v = (np.arange(32, dtype=np.float32) - 16.0) * 0.5
    blk = orc.quantize_q4(v.reshape(1, 32))[0, 0]
    scale = blk[:4].view(np.float32)[0]
    deq = np.empty(32, np.float32)
    for i in range(16):
        deq[2 * i] = (int(blk[4 + i] & 0xF) - 8) * scale
        deq[2 * i + 1] = (int(blk[4 + i] >> 4) - 8) * scale
    assert np.all(np.abs(v - deq) < 2.0)


def test_ref_q4_matvec(orc):
    """src/quantize.rs:2274-2289: 2x32 matrix with single ones, x = (5, 3, 0...)."""
    W = np.zeros((2, 32), np.float32)
    W[0, 0] = 1.0
    W[1, 1] = 1.0
    x = np.zeros(32, np.float32)
    x[0], x[1] = 5.0, 3.0
    for order in ("scalar", "avx2"):
        y = orc.q4_matvec(orc.quantize_q4(W), x, order=order)
        assert abs(y[0] - 5.0) < 2.0 and abs(y[1] - 3.0) < 2.0
        # known answer: amax 1 -> scale 1/7, q = 7 -> dequantised weight 7 * f32(1/7)
        assert y[0] == np.float32(7.0) * (np.float32(1.0) / np.float32(7.0)) * np.float32(5.0)


def test_ref_awq_scaling(orc):
    """src/quantize.rs:2522-2546: uniform AWQ scales leave the product approximately unchanged."""
    W = np.concatenate([(np.arange(32) - 16.0) * 0.3, (np.arange(32) - 16.0) * 0.1]).astype(np.float32).reshape(2, 32)
    x = np.ones(32, np.float32)
    y0 = orc.q4_matvec(orc.quantize_q4(W), x)
    Wb = orc.from_act16(orc.to_act16(W, True), True)  # the reference quantises from a bf16 tensor here
    awq = np.full(32, 1.5, np.float32)
    y1 = orc.q4_matvec(orc.quantize_q4(Wb, awq), x, orc.awq_inverse(awq))
    assert np.all(np.abs(y0 - y1) < 5.0)
    assert np.all(np.abs(y0 - y1) < 0.5)  # much tighter in practice


# ------------------------------------------------------------------ hand-computed known answers
def test_kat_weight_blocks(orc, golden):
    nib, sc = golden["w_edge_nibbles"], golden["w_edge_scales"]
    q = npo.unpack_gpu(nib)  # signed values
    # all-zero block: scale 0, every value 0 (nibble 8)
    assert sc[0, 0] == 0.0 and np.all(q[0, 0:32] == 0)
    # single +amax: scale amax/7, that element 7, the rest 0
    assert sc[1, 1] == np.float32(0.0625) / np.float32(7.0)
    assert q[1, 32 + 5] == 7 and np.count_nonzero(q[1, 32:64]) == 1
    # exact ties with scale 1: half away from zero
    assert sc[3, 2] == 1.0
    assert list(q[3, 64:80]) == [1, -1, 2, -2, 3, -3, 4, -4, 5, -5, 6, -6, 7, -7, 7, -7]
    # -amax maps to -7: for a finite 1/scale the value -8 (nibble 0) is never produced
    rows = [r for r in range(16) if r != 4]
    assert q[5, 96] == -7 and q[rows].min() >= -7 and q.max() <= 7
    # subnormal amax: 1/scale overflows to +inf, v*inf = +-inf saturates through the i8 cast to 127 / -128,
    # then clamps to 7 / -8 -- the only way the reference quantizer emits nibble 0
    w4 = golden["w_edge"][4, 0:32]
    assert np.array_equal(q[4, 0:32], np.where(w4 > 0, 7, -8))


def test_kat_activation_groups(orc, golden):
    xq, xs = golden["act_f16_q"], golden["act_f16_s"]
    assert xs[0] == 1.0 and np.all(xq[0:32] == 0)  # zero group: scale 1
    assert xs[1] == 1.0
    # ties to even: 0.5->0, 1.5->2, 2.5->2, -0.5->0, -1.5->-2, -2.5->-2, 3.5->4, -3.5->-4, 126.5->126, ..., 127
    assert list(xq[32:44]) == [0, 2, 2, 0, -2, -2, 4, -4, 126, -126, 127, -127]
    assert xq.min() >= -127  # -128 is never produced


def test_dp4a_formulation_matches_signed_dot(orc, golden):
    """sum(raw_nibble * xq) - 8 * sum(xq) over the {j, j+16} byte layout equals sum((q-8) * xq)."""
    nib, xq = golden["g_nibbles"].astype(np.int64), golden["g_xq"].astype(np.int64)
    N, half = nib.shape
    nb = half // 16
    raw = nib.reshape(N, nb, 16)
    x = xq.reshape(nb, 32)
    lo = (raw & 0xF) * x[None, :, :16]
    hi = (raw >> 4) * x[None, :, 16:]
    I = lo.sum(2) + hi.sum(2) - 8 * x.sum(1)[None, :]
    assert np.array_equal(I.astype(np.int32), golden["g_idot"])
    assert np.abs(golden["g_idot"]).max() <= 32 * 8 * 127


# ------------------------------------------------------------------ cross-checks
def test_generator_matches_numpy(orc):
    a = orc.fill_normal(4096, 77, 3, first=11, scale=0.02)
    assert same_bits(a, npo.fill_normal(4096, 77, 3, first=11, scale=0.02))
    assert same_bits(orc.fill_uniform(4096, 77, 3, first=11), npo.fill_uniform(4096, 77, 3, first=11))
    z = orc.fill_normal(200000, 1, 1)
    assert abs(z.mean()) < 0.01 and abs(z.std() - 1.0) < 0.01


def test_oracle_matches_numpy_random(orc):
    rng = np.random.default_rng(5)
    for (N, K) in [(1, 32), (5, 64), (33, 416), (64, 2048)]:
        W = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
        x16 = orc.to_act16(rng.standard_normal(K).astype(np.float32))
        nib, sc = orc.extract_for_gpu(orc.quantize_q4(W))
        q, s2 = npo.quantize_q4(W)
        assert same_bits(npo.pack_gpu(q), nib) and same_bits(s2, sc)
        xq, xs = orc.quantize_q8(x16)
        xq2, xs2 = npo.quantize_q8(orc.from_act16(x16))
        assert same_bits(xq, xq2) and same_bits(xs, xs2)
        assert same_bits(orc.w4a8_idot(xq, nib), npo.w4a8_idot(xq, nib))
        y = orc.w4a16_matvec_f64(orc.from_act16(x16), nib, sc)
        assert np.allclose(y, npo.w4a16_matvec(orc.from_act16(x16), nib, sc), rtol=0, atol=1e-12)


def test_cpu_orders_agree_within_rounding(orc, golden):
    y0, y1, y64 = golden["g_y_cpu_scalar"], golden["g_y_cpu_avx2"], golden["g_y_w4a16_f64"]
    rms = np.sqrt(np.mean(y64**2))
    assert np.max(np.abs(y0 - y64)) / rms < 1e-5 and np.max(np.abs(y1 - y64)) / rms < 1e-5


def test_threaded_baseline_matches_serial(orc, golden):
    orc.set_threads(4)
    xf = orc.from_act16(golden["g_x16"])
    y_mt = orc.q4_matvec_mt(golden["g_blocks"], xf)
    ref = golden["g_y_cpu_avx2"] if orc.have_avx2() else golden["g_y_cpu_scalar"]
    assert same_bits(y_mt, ref)
    y8 = orc.w4a8_matvec_mt(golden["g_xq"], golden["g_xs"], golden["g_nibbles"], golden["g_scales"])
    assert np.max(np.abs(y8 - golden["g_y_w4a8_f64"])) < 1e-4 * np.sqrt(np.mean(golden["g_y_w4a8_f64"] ** 2))
    orc.set_threads(1)


def test_f16_conversions_match_numpy(orc):
    rng = np.random.default_rng(3)
    t = (rng.standard_normal(50000) * 10.0 ** rng.integers(-9, 5, 50000)).astype(np.float32)
    assert same_bits(orc.f32_to_f16_bits(t), t.astype(np.float16).view(np.uint16))
    allh = np.arange(65536, dtype=np.uint16)
    fin = ~np.isnan(allh.view(np.float16))
    assert same_bits(orc.f16_bits_to_f32(allh)[fin], allh.view(np.float16).astype(np.float32)[fin])


def test_rms_norm_orders(orc, golden):
    ref = golden["n_out_f64"]
    got = orc.from_act16(golden["n_out16"])
    assert np.max(np.abs(got - ref)) <= 2e-3 * np.max(np.abs(ref))  # one f16 rounding
    assert np.allclose(npo.rms_norm(orc.from_act16(golden["n_x16"]), orc.from_act16(golden["n_w16"]), 1e-5), ref)


def test_routing_predicate(orc):
    assert orc.use_w4a8(0.0) and orc.use_w4a8(0.69999) and not orc.use_w4a8(0.7) and not orc.use_w4a8(1.0)
    assert not orc.use_w4a8(0.0, no_w4a8=True)
    assert list(orc.normalize_importance([3.0, 3.0, 3.0])) == [0.5, 0.5, 0.5]
    assert list(orc.normalize_importance([1.0, 2.0, 3.0])) == [0.0, 0.5, 1.0]
