"""The persistent whole-step kernel (nve_b200_decode_step) against the six-launch-per-layer graph.

Both run the same device functions in the same order, so hidden states, KV caches and logits must agree bit for
bit on every shape; the six-launch path is itself checked against the oracle in test_gpu_glue.py.
"""
import numpy as np
import pytest

from helpers import TOL, dev, rel_rms_err

pytestmark = pytest.mark.gpu


def _state(torch, hidden, ffn, nh, nkv, hd, layers, max_seq, seed, norm_jitter=True, awq=False):
    from nve_b200 import cuda_kernels as ck
    from nve_b200.bench_random import rope_tables
    from nve_b200.gpu_layer import GpuInferenceState, GpuKvCache, GpuLayerWeights, GpuW4, RoutingConfig

    def w4(n, k, sid, a=None):
        W = ck.fill_normal(n * k, seed, sid, scale=0.02).view(n, k)
        nib, sc = ck.q4_quantize(W)
        return GpuW4(nib, sc, a, n, k)

    def vec(n, sid, base=1.0, amp=0.1):
        return (base + amp * ck.fill_normal(n, seed, sid)).to(torch.float16)

    lw = []
    for li in range(layers):
        b = 100 * li
        a_h = (1.0 + 0.2 * ck.fill_normal(hidden, seed, b + 50)).abs() if awq else None
        a_o = (1.0 + 0.2 * ck.fill_normal(nh * hd, seed, b + 51)).abs() if awq else None
        a_f = (1.0 + 0.2 * ck.fill_normal(hidden, seed, b + 52)).abs() if awq else None
        a_d = (1.0 + 0.2 * ck.fill_normal(ffn, seed, b + 53)).abs() if awq else None
        n1 = vec(hidden, b + 60) if norm_jitter else torch.ones(hidden, dtype=torch.float16, device="cuda")
        n2 = vec(hidden, b + 61) if norm_jitter else torch.ones(hidden, dtype=torch.float16, device="cuda")
        lw.append(GpuLayerWeights(w4(nh * hd, hidden, b + 1, a_h), w4(nkv * hd, hidden, b + 2, a_h),
                                  w4(nkv * hd, hidden, b + 3, a_h), w4(hidden, nh * hd, b + 4, a_o),
                                  w4(ffn, hidden, b + 5, a_f), w4(ffn, hidden, b + 6, a_f), w4(hidden, ffn, b + 7, a_d),
                                  n1, n2))
    kv = GpuKvCache(layers, nkv, max_seq, hd, "cuda")
    cos, sin = rope_tables(hd, max_seq, 10000.0, "cuda")
    return GpuInferenceState(lw, kv, nh, nkv, hd, 1e-5, cos, sin, RoutingConfig(False, 0.7), True)


def _fill_kv(torch, st, seed, upto):
    from nve_b200 import cuda_kernels as ck

    for li in range(len(st.layer_weights)):
        for t, sid in ((st.kv_cache.k[li], 7000 + 2 * li), (st.kv_cache.v[li], 7001 + 2 * li)):
            r = ck.fill_normal(t.numel(), seed, sid, dtype=torch.float16).view_as(t)
            t[:, :upto].copy_(r[:, :upto])


SHAPES = [
    # hidden, ffn, nh, nkv, hd, layers, max_seq, start_pos
    (512, 1024, 8, 2, 64, 4, 16, 0),        # K = 512 / 1024: one and one column set, positions from 0
    (2048, 8192, 32, 8, 64, 2, 96, 40),     # Llama-3.2-1B layer shape
    (4096, 14336, 32, 8, 128, 2, 300, 257),  # Llama-3.1-8B layer shape, ragged position slices
    (1024, 3584, 16, 2, 128, 3, 64, 63),    # 8 query heads per KV head, K = 3584 (3.5 column sets), last position
]


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("awq", [False, True])
def test_persistent_step_equals_six_launch_graph(cuda, shape, awq):
    from nve_b200 import cuda_kernels as ck
    from nve_b200.decode_graph import PersistentDecode, StaticDecodeGraph

    torch = cuda
    hidden, ffn, nh, nkv, hd, layers, max_seq, pos0 = shape
    imp = [0.1, 0.9, 0.4, 1.0][:layers]  # threshold 0.7: W4A8, W4A16, W4A8, W4A16
    st_g = _state(torch, hidden, ffn, nh, nkv, hd, layers, max_seq, 311, awq=awq)
    st_p = _state(torch, hidden, ffn, nh, nkv, hd, layers, max_seq, 311, awq=awq)
    _fill_kv(torch, st_g, 312, pos0)
    _fill_kv(torch, st_p, 312, pos0)
    steps = min(3, max_seq - pos0)
    inputs = [ck.fill_normal(hidden, 313, s, dtype=torch.float16).view(1, -1) for s in range(steps)]

    graph = StaticDecodeGraph(st_g, hidden, ffn, imp)
    with ck.attn_decode_kernel(cuda_core=True):  # the persistent kernel's attention phase shares that kernel's arithmetic
        graph.capture()
    want = []
    try:
        for s in range(steps):
            want.append(graph.replay(inputs[s], pos0 + s))
            torch.cuda.synchronize()  # the next replay rewrites the pinned position scalars this one reads
    finally:
        graph.destroy()

    pers = PersistentDecode(st_p, hidden, ffn, imp)
    assert pers.routes == graph.routes
    pers.capture()
    try:
        for s in range(steps):
            got = pers.replay(inputs[s], pos0 + s)
            torch.cuda.synchronize()
            assert pers.error() == 0
            assert torch.isfinite(got.float()).all()
            assert torch.equal(got, want[s]), f"step {s}: hidden state differs from the six-launch graph"
    finally:
        pers.destroy()
    for li in range(layers):
        assert torch.equal(st_g.kv_cache.k[li], st_p.kv_cache.k[li])
        assert torch.equal(st_g.kv_cache.v[li], st_p.kv_cache.v[li])


def test_persistent_step_eager_launch_and_prefetch_off(cuda):
    """The kernel launched directly (no graph) with device position scalars, with and without the L2 prefetch
    stream: same bits."""
    from nve_b200 import cuda_kernels as ck
    from nve_b200.decode_graph import PersistentDecode

    torch = cuda
    hidden, ffn, nh, nkv, hd, layers, max_seq, pos = 2048, 8192, 32, 8, 64, 2, 64, 33
    imp = [0.1, 0.9]
    outs = []
    old = ck.decode_step_set_prefetch(-1)
    try:
        for pf in (old, 0):
            ck.decode_step_set_prefetch(pf)
            st = _state(torch, hidden, ffn, nh, nkv, hd, layers, max_seq, 411)
            _fill_kv(torch, st, 412, pos)
            pers = PersistentDecode(st, hidden, ffn, imp)
            st.set_position(pos)
            pers.hidden_buf.copy_(ck.fill_normal(hidden, 413, 0, dtype=torch.float16).view(1, -1))
            pers.step(st.d_pos.data_ptr(), st.d_seqlen.data_ptr())
            torch.cuda.synchronize()
            assert pers.error() == 0
            outs.append(pers.hidden_buf.clone())
    finally:
        ck.decode_step_set_prefetch(old)
    assert torch.equal(outs[0], outs[1])


def test_persistent_step_lm_head(cuda, orc):
    """Final RMSNorm + lm_head inside the kernel == nve_b200_rmsnorm_matvec_* on the final hidden state, and within
    tolerance of the oracle's f64 W4A16 GEMV on the normalised row."""
    from nve_b200 import cuda_kernels as ck
    from nve_b200.decode_graph import PersistentDecode
    from nve_b200.gpu_layer import GpuW4

    torch = cuda
    hidden, ffn, nh, nkv, hd, layers, max_seq, pos, vocab = 1024, 2048, 8, 2, 128, 2, 32, 9, 5000
    imp = [0.1, 0.9]
    W = ck.fill_normal(vocab * hidden, 511, 900, scale=0.02).view(vocab, hidden)
    nib, sc = ck.q4_quantize(W)
    lm = GpuW4(nib, sc, None, vocab, hidden)
    fnorm = (1.0 + 0.1 * ck.fill_normal(hidden, 511, 901)).to(torch.float16)
    for use_w4a8 in (False, True):
        st = _state(torch, hidden, ffn, nh, nkv, hd, layers, max_seq, 512)
        _fill_kv(torch, st, 513, pos)
        pers = PersistentDecode(st, hidden, ffn, imp, lm_head=(lm, fnorm, use_w4a8))
        pers.capture()
        try:
            h = pers.replay(ck.fill_normal(hidden, 514, 0, dtype=torch.float16).view(1, -1), pos)
            torch.cuda.synchronize()
            assert pers.error() == 0
        finally:
            pers.destroy()
        if use_w4a8:
            want = ck.rmsnorm_matvec_w4a8_multi(h, fnorm, 1e-5, [lm.triple()], hidden, out_dtype=torch.float32)[0]
        else:
            want = ck.rmsnorm_matvec_w4a16_multi(h, fnorm, 1e-5, None, [lm.triple()], hidden, out_dtype=torch.float32)[0]
        assert torch.equal(pers.logits.view(-1), want.view(-1))
        if not use_w4a8:
            normed = ck.fused_rms_norm(h, fnorm, 1e-5)
            ref = orc.w4a16_matvec_f64(normed.float().cpu().numpy().reshape(-1), nib.cpu().numpy(), sc.cpu().numpy())
            assert rel_rms_err(pers.logits.cpu().numpy(), ref) < TOL


def test_bounded_wait_reports_timeout_instead_of_hanging(cuda):
    """A wait that nothing will ever satisfy (one CTA at a barrier for two) gives up after its time limit and latches
    NVE_ERR_TIMEOUT; the context stays usable and the workspace works again after a reset."""
    from nve_b200 import cuda_kernels as ck

    torch = cuda
    ws = torch.zeros(4096 + 256, dtype=torch.uint8, device="cuda")
    ws = ws[(-ws.data_ptr()) % 256:][:4096]
    ck.decode_step_init(ws)
    assert ck.decode_step_error(ws) == 0
    ck.decode_step_wait_probe(ws, 2_000_000)  # 2 ms
    torch.cuda.synchronize()
    assert ck.decode_step_error(ws, reset=True) == 7  # NVE_ERR_TIMEOUT
    assert ck.decode_step_error(ws) == 0
    assert int(ws.view(torch.int64)[0].item()) == 0  # barrier counter cleared with the error word
    x = torch.ones(4, device="cuda")
    assert float(x.sum().item()) == 4.0
