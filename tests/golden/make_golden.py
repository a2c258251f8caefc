"""Generates the golden fixtures in this directory (run from the repository root:
``python tests/golden/make_golden.py``).

The reference's CPU path is Rust and cannot be built or imported where these fixtures are made, so the
expected values come from the C oracle (oracle/nve_oracle.c) and are accepted only when the independent
numpy restatement (oracle/np_oracle.py) produces the same bits.  Inputs come from the shared counter-based
generator plus hand-built edge blocks; every array needed to replay a case is stored, so the tests do not
depend on the generator.
"""
from __future__ import annotations

import hashlib
import os
import sys

import numpy as np

sys.path.insert(0, os.path.abspath(os.path.join(os.path.dirname(__file__), "..", "..")))
import oracle as o  # noqa: E402
from oracle import np_oracle as npo  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
SEED = 20240607


def _same_bits(a, b):
    return a.shape == b.shape and a.dtype == b.dtype and a.tobytes() == b.tobytes()


def weight_edge_matrix() -> np.ndarray:
    """16 x 128 weights ~N(0, 0.02) with hand-built edge blocks."""
    W = o.fill_normal(16 * 128, SEED, 1, scale=0.02).reshape(16, 128).copy()
    W[0, 0:32] = 0.0                                   # all-zero block: scale 0, every nibble 8
    W[1, 32:64] = 0.0
    W[1, 32 + 5] = 0.0625                              # single +amax
    W[2, 0:32] = (np.arange(32, dtype=np.float32) - 16.0) * 0.5   # the reference's round-trip vector
    t = np.zeros(32, np.float32)                       # amax 7 -> scale 1: exact ties, half away from zero
    t[:14] = [0.5, -0.5, 1.5, -1.5, 2.5, -2.5, 3.5, -3.5, 4.5, -4.5, 5.5, -5.5, 6.5, -6.5]
    t[14], t[15] = 7.0, -7.0
    W[3, 64:96] = t
    W[4, 0:32] = np.float32(1e-40) * np.sign(W[4, 0:32] + 1e-30)  # subnormal amax
    W[5, 96:128] = 0.01
    W[5, 96] = -0.07                                   # -amax -> q = -7 -> nibble 1 (nibble 0 unreachable)
    W[6, 0:32] = np.float32(3.0e38) * np.where(np.arange(32) % 2 == 0, 1, -1)  # near f32 max
    return W


def act_edge_vector(bf16: bool) -> np.ndarray:
    """256 activations ~N(0,1) with hand-built edge groups, returned as 16-bit patterns."""
    x = o.fill_normal(256, SEED, 2).copy()
    x[0:32] = 0.0                                      # zero group: scale 1, codes 0
    g = np.zeros(32, np.float32)                       # amax 127 -> scale 1: ties go to even
    g[:12] = [0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 3.5, -3.5, 126.5, -126.5, 127.0, -127.0]
    x[32:64] = g
    x[64:96] = np.float32(6e-8) * (np.arange(32) - 15.5)   # f16 subnormal range (flushes to 0 or tiny in f16)
    x[96:128] = 60000.0 * np.where(np.arange(32) % 3 == 0, -1.0, 0.37)
    return o.to_act16(x, bf16)


def main() -> None:
    out = {}
    # ---- case 1: weight quantizer and the two packings
    W = weight_edge_matrix()
    blocks = o.quantize_q4(W)
    nib, sc = o.extract_for_gpu(blocks)
    q, s2 = npo.quantize_q4(W)
    assert _same_bits(npo.pack_cpu(q, s2), blocks) and _same_bits(npo.pack_gpu(q), nib) and _same_bits(s2, sc)
    out.update(w_edge=W, w_edge_blocks=blocks, w_edge_nibbles=nib, w_edge_scales=sc)

    # ---- case 2: activation quantizer, f16 and bf16
    for tag, bf in (("f16", False), ("bf16", True)):
        x16 = act_edge_vector(bf)
        xq, xs = o.quantize_q8(x16, bf)
        xq2, xs2 = npo.quantize_q8(o.from_act16(x16, bf))
        assert _same_bits(xq, xq2) and _same_bits(xs, xs2)
        out[f"act_{tag}"] = x16
        out[f"act_{tag}_q"] = xq
        out[f"act_{tag}_s"] = xs

    # ---- case 3: GEMVs on 64 x 256 (rows include the edge rows above, tiled)
    Wg = o.fill_normal(64 * 256, SEED, 3, scale=0.02).reshape(64, 256).copy()
    Wg[:16, :128] = W
    gb = o.quantize_q4(Wg)
    gn, gs = o.extract_for_gpu(gb)
    x16 = act_edge_vector(False)
    x16[64:128] = o.to_act16(o.fill_normal(64, SEED, 4))  # keep magnitudes sane for the dot products
    xf = o.from_act16(x16)
    xq, xs = o.quantize_q8(x16)
    idot = o.w4a8_idot(xq, gn)
    assert _same_bits(idot, npo.w4a8_idot(xq, gn))
    y8 = o.w4a8_matvec_f64(xq, xs, gn, gs)
    assert np.allclose(y8, npo.w4a8_matvec(xq, xs, gn, gs), rtol=0, atol=1e-12)
    y16 = o.w4a16_matvec_f64(xf, gn, gs)
    assert np.allclose(y16, npo.w4a16_matvec(xf, gn, gs), rtol=0, atol=1e-12)
    awq = (1.0 + 0.5 * o.fill_uniform(256, SEED, 5)).astype(np.float32)
    gb_awq = o.quantize_q4(Wg, awq)
    gn_awq, gs_awq = o.extract_for_gpu(gb_awq)
    awq_inv = o.awq_inverse(awq)
    out.update(
        g_w=Wg, g_blocks=gb, g_nibbles=gn, g_scales=gs, g_x16=x16, g_xq=xq, g_xs=xs, g_idot=idot,
        g_y_w4a8_f64=y8, g_y_w4a8_b200=o.w4a8_matvec_b200(xq, xs, gn, gs),
        g_y_w4a8_reforder=o.w4a8_matvec_reforder(xq, xs, gn, gs),
        g_y_cpu_scalar=o.q4_matvec(gb, xf, order="scalar"), g_y_cpu_avx2=o.q4_matvec(gb, xf, order="avx2"),
        g_y_w4a16_f64=y16, g_y_w4a16_b200=o.w4a16_matvec_b200(x16, gn, gs),
        g_awq=awq, g_awq_inv=awq_inv, g_awq_nibbles=gn_awq, g_awq_scales=gs_awq,
        g_y_awq_cpu_scalar=o.q4_matvec(gb_awq, xf, awq_inv, order="scalar"),
        g_y_awq_f64=o.w4a16_matvec_f64(xf, gn_awq, gs_awq, awq_inv),
        g_y_awq_b200=o.w4a16_matvec_b200(x16, gn_awq, gs_awq, awq_inv),
    )

    # ---- case 4: glue (RMSNorm in the library's order, SiLU*up, routing)
    h = o.fill_normal(512, SEED, 6)
    h16 = o.to_act16(h)
    w16 = o.to_act16(1.0 + 0.1 * o.fill_normal(512, SEED, 7))
    out.update(n_x16=h16, n_w16=w16, n_out16=o.rms_norm_16(h16, w16, 1e-5),
               n_out_f64=o.rms_norm_f64(o.from_act16(h16), o.from_act16(w16), 1e-5))
    scores = o.fill_uniform(32, SEED, 8).astype(np.float64)
    out.update(r_scores=scores, r_norm=o.normalize_importance(scores))

    # ---- case 5: measurement configuration 1 (W4A16 GEMV, Llama-3.2-1B up_proj 8192 x 2048), digest + head only
    Wc = o.fill_normal(8192 * 2048, SEED, 10, scale=0.02).reshape(8192, 2048)
    xc = o.fill_normal(2048, SEED, 11)
    cb = o.quantize_q4(Wc)
    cn, cs = o.extract_for_gpu(cb)
    xc16 = o.to_act16(xc)
    yc = o.q4_matvec(cb, o.from_act16(xc16), order="scalar")
    ycb = o.w4a16_matvec_b200(xc16, cn, cs)
    out.update(
        c1_nibbles_sha=np.frombuffer(hashlib.sha256(cn.tobytes()).digest(), np.uint8),
        c1_scales_sha=np.frombuffer(hashlib.sha256(cs.tobytes()).digest(), np.uint8),
        c1_y_cpu_scalar_sha=np.frombuffer(hashlib.sha256(yc.tobytes()).digest(), np.uint8),
        c1_y_b200_sha=np.frombuffer(hashlib.sha256(ycb.tobytes()).digest(), np.uint8),
        c1_y_cpu_scalar_head=yc[:64].copy(), c1_y_b200_head=ycb[:64].copy(),
        c1_y_rms=np.array([np.sqrt((yc.astype(np.float64) ** 2).mean())]),
    )
    path = os.path.join(HERE, "decode_path_golden.npz")
    np.savez_compressed(path, seed=np.array([SEED]), **out)
    print(f"wrote {path}: {os.path.getsize(path)} bytes, {len(out)} arrays")


if __name__ == "__main__":
    main()
