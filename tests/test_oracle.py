"""The CPU oracle against the reference's own known-answer tests.

Each case restates one of the hot-path test binaries of the reference
(crates/oxide-infer-server/src/bin/*.rs) with the same generator, shapes,
windows and tolerances; the kernels under test there are replaced by the
oracle's restatement of them.
"""
import numpy as np
import pytest

from oracle import cpu as O

NQ, NKV, HD = O.NQ, O.NKV, O.HD


def test_f16_conversion_matches_numpy():
    rng = np.random.default_rng(0)
    x = np.concatenate([
        rng.standard_normal(200000).astype(np.float32) * 3,
        (rng.standard_normal(50000) * 1e-5).astype(np.float32),
        (rng.standard_normal(50000) * 1e-7).astype(np.float32),
        np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e9, -1e9, 2.0 ** -24, 2.0 ** -25,
                  np.nextafter(np.float32(2.0 ** -25), np.float32(1)), 2.0 ** -14, np.inf, -np.inf],
                 np.float32),
    ])
    got = O.f2h(x).view(np.uint16)
    with np.errstate(over="ignore"):
        want = x.astype(np.float16).view(np.uint16)
    assert np.array_equal(got, want)
    # and back: every finite half value round-trips exactly
    allh = np.arange(65536, dtype=np.uint16)
    L = O.lib()
    back = np.array([L.orc_h2f(int(h)) for h in allh[::7]], np.float32)
    ref = allh[::7].view(np.float16).astype(np.float32)
    ok = np.isnan(ref) | (back == ref)
    assert ok.all()


def test_pat_generator():
    # test_split_attention.rs:28-34
    a = O.pat(3, 5000)
    b = O.pat_numpy(3, 5000)
    assert np.array_equal(a, b)
    assert a.min() >= -1.0 and a.max() <= 1.0


def _one_row(q, k, v, slen, window):
    kp, vp = O.ptr_table([k]), O.ptr_table([v])
    sl = np.array([slen], np.uint32)
    return kp, vp, sl


def test_uniform_softmax_mean_position():
    """debug_online_attn.rs:1-5: q = k = 1, v[t] = t => output = mean kept position."""
    seq = 300
    q = np.ones((1, NQ, HD), np.float16)
    k = np.ones((seq, NKV, HD), np.float16)
    v = np.broadcast_to(np.arange(seq, dtype=np.float16)[:, None, None], (seq, NKV, HD)).copy()
    kp, vp, sl = _one_row(q, k, v, seq, 0)
    for window, want in [(0, 149.5), (256, (44 + 299) / 2)]:
        for fn in (O.attn_online, lambda *a: O.attn_combine(*O.attn_split(*a))):
            got = fn(q, kp, vp, sl, window).astype(np.float32)
            assert np.abs(got - want).max() <= 0.05, (window, got.min(), got.max())


@pytest.mark.parametrize("window", [0, 512, 300, 257, 256, 128])
def test_sliding_window_boundary(window):
    """test_swa_attention.rs: 300 keys, key masked iff p_q - p_k >= window; < 2e-3 vs f64."""
    seq = 300
    qf = O.pat(1, NQ * HD)
    kf = O.pat(2, seq * NKV * HD, 2.0)
    vf = O.pat(3, seq * NKV * HD)
    q = O.f2h(qf).reshape(1, NQ, HD)
    k, v = O.f2h(kf), O.f2h(vf)
    kp, vp, sl = _one_row(q, k, v, seq, window)
    want = O.attention_f64(qf, kf, vf, seq, window)
    got = O.attn_online(q, kp, vp, sl, window)[0].astype(np.float64)
    assert np.abs(got - want).max() < 2e-3
    got2 = O.attn_combine(*O.attn_split(q, kp, vp, sl, window))[0].astype(np.float64)
    assert np.abs(got2 - want).max() < 2e-3


@pytest.mark.parametrize("window", [0, 256])
def test_split_combine_rows(window):
    """test_split_attention.rs: rows 300/180/64/300, own Q and KV, K x2; < 3e-3 each way."""
    rows = [300, 180, 64, 300]
    max_seq = 300
    qf = O.pat(1, len(rows) * NQ * HD).reshape(len(rows), NQ, HD)
    ks = [O.pat(2 + r, max_seq * NKV * HD, 2.0) for r in range(len(rows))]
    vs = [O.pat(9 + r, max_seq * NKV * HD) for r in range(len(rows))]
    q = O.f2h(qf)
    kh, vh = [O.f2h(a) for a in ks], [O.f2h(a) for a in vs]
    kp, vp = O.ptr_table(kh), O.ptr_table(vh)
    sl = np.array(rows, np.uint32)
    acc, stats = O.attn_split(q, kp, vp, sl, window)
    # grid sizing mirrors the engine: ceil(min(slen, window)/128) maximised over rows
    assert acc.shape[1] == (3 if window == 0 else 2)
    split = O.attn_combine(acc, stats).astype(np.float64)
    online = O.attn_online(q, kp, vp, sl, window).astype(np.float64)
    for r, slen in enumerate(rows):
        want = O.attention_f64(qf[r], ks[r], vs[r], slen, window)
        assert np.abs(split[r] - want).max() < 3e-3
        assert np.abs(online[r] - want).max() < 3e-3
        assert np.abs(split[r] - online[r]).max() < 3e-3


@pytest.mark.parametrize("window", [0, 256])
def test_gemm_prefill_chunks(window):
    """test_gemm_attention.rs: chunks {96 rows @p0=0, 128 rows @p0=400}, cache 600;
    GEMM path vs online+gate <= 8e-3, vs f64 on first/last row <= 2e-2."""
    cache_len = 600
    chunks = [(0, 96, 0), (96, 128, 400)]
    total = sum(c[1] for c in chunks)
    qf = O.pat(1, total * NQ * HD).reshape(total, NQ, HD)
    gf = O.pat(7, total * NQ, 2.0).reshape(total, NQ)
    q, g = O.f2h(qf), O.f2h(gf)
    for ci, (start, rows, p0) in enumerate(chunks):
        kf = O.pat(20 + ci, cache_len * NKV * HD, 1.5)
        vf = O.pat(40 + ci, cache_len * NKV * HD)
        k, v = O.f2h(kf), O.f2h(vf)
        qs, gs = q[start:start + rows].copy(), g[start:start + rows].copy()
        got = O.prefill_gemm_chunk(qs, gs, k, v, p0, window).astype(np.float64)
        kp = np.full(rows, k.ctypes.data, np.uint64)
        vp = np.full(rows, v.ctypes.data, np.uint64)
        sl = (p0 + 1 + np.arange(rows)).astype(np.uint32)
        online = O.attn_online(qs, kp, vp, sl, window)
        gsig = 1.0 / (1.0 + np.exp(-gs.astype(np.float32)))
        want_online = online.astype(np.float32) * gsig[:, :, None]
        assert np.abs(got - want_online).max() <= 8e-3
        for r in (0, rows - 1):
            want = O.attention_f64(qf[start + r], kf, vf, p0 + r + 1, window,
                                   gate=gs[r].astype(np.float32))
            assert np.abs(got[r] - want).max() <= 2e-2


def test_conv_unit_weights_zero_state():
    """kernels/src/conv.rs:224-268: zero state, weights 1, input 2 => output 2.0."""
    hidden, b = 2048, 3
    state = [np.zeros((hidden, 6), np.float16) for _ in range(b)]
    bcx = np.empty((b, 3 * hidden), np.float16)
    bcx[:, :hidden] = 1.0          # B
    bcx[:, hidden:2 * hidden] = 1.0  # C
    bcx[:, 2 * hidden:] = 2.0      # x
    w = np.ones((hidden, 7), np.float16)
    y = O.conv_decode(O.ptr_table(state), bcx, w)
    assert np.all(y.astype(np.float32) == 2.0)
    for s in state:
        assert np.all(s[:, :5] == 0) and np.all(s[:, 5].astype(np.float32) == 2.0)


def test_conv_prefill_equals_tokenwise_decode():
    """The wave path (gather + conv + copy-back) must leave the same y and the
    same persistent state as feeding the chunk one token at a time through the
    decode kernel: both are reference paths for the same recurrence."""
    rng = np.random.default_rng(1)
    hidden = 2048
    lens = [1, 5, 6, 7, 19]
    rows = sum(lens)
    bcx = rng.standard_normal((rows, 3 * hidden)).astype(np.float16)
    w = (rng.standard_normal((hidden, 7)) * 0.1).astype(np.float16)
    carry0 = [rng.standard_normal((hidden, 6)).astype(np.float16) for _ in lens]
    origin, lpos, carry_rows = [], [], []
    a = [c.copy() for c in carry0]
    r0 = 0
    for i, n in enumerate(lens):
        origin += [r0] * n
        lpos += list(range(n))
        carry_rows += [a[i]] * n
        r0 += n
    y_wave = O.conv_prefill_wave(O.ptr_table(carry_rows), np.array(origin, np.uint32),
                                 np.array(lpos, np.uint32), bcx, w)
    b = [c.copy() for c in carry0]
    y_seq = np.empty_like(y_wave)
    r = 0
    for i, n in enumerate(lens):
        for _ in range(n):
            y_seq[r] = O.conv_decode(O.ptr_table([b[i]]), bcx[r:r + 1].copy(), w)[0]
            r += 1
    assert np.array_equal(y_wave.view(np.uint16), y_seq.view(np.uint16))
    for x, z in zip(a, b):
        assert np.array_equal(x.view(np.uint16), z.view(np.uint16))


def test_rmsnorm_rope_against_f64_model():
    rng = np.random.default_rng(2)
    b = 5
    x = rng.standard_normal((b, NQ, HD)).astype(np.float16)
    w = (1 + 0.02 * rng.standard_normal(HD)).astype(np.float16)
    pos = np.array([0, 1, 77, 4095, 8191], np.uint32)
    cos, sin = O.rope_table(8192, 1e6, 0.5)
    # partial rotary 0.5: dims 32..63 and 96..127 are identity (rope.rs:166-170)
    assert np.all(cos[:, 32:64].astype(np.float32) == 1) and np.all(sin[:, 96:].astype(np.float32) == 0)
    got = x.copy()
    O.qk_rmsnorm(got, w)
    xf = x.astype(np.float64)
    normed = xf / np.sqrt((xf ** 2).mean(-1, keepdims=True) + 1e-5) * w.astype(np.float64)
    n16 = got.astype(np.float64)
    assert np.abs(n16 - normed).max() < 4e-3  # one f16 ulp at |x|<4
    O.rope(got, cos, sin, pos)
    c, s = cos[pos].astype(np.float64)[:, None], sin[pos].astype(np.float64)[:, None]
    rot = np.concatenate([-n16[..., 64:], n16[..., :64]], -1)
    want = n16 * c + rot * s
    assert np.abs(got.astype(np.float64) - want).max() < 4e-3


def test_kv_copy_and_decode_layer_append_position():
    rng = np.random.default_rng(3)
    b = 4
    lens = np.array([5, 130, 257, 64], np.uint32)
    ks = [rng.standard_normal((int(n) + 1, NKV, HD)).astype(np.float16) for n in lens]
    vs = [rng.standard_normal((int(n) + 1, NKV, HD)).astype(np.float16) for n in lens]
    q = rng.standard_normal((b, NQ, HD)).astype(np.float16)
    k = rng.standard_normal((b, NKV, HD)).astype(np.float16)
    v = rng.standard_normal((b, NKV, HD)).astype(np.float16)
    gate = rng.standard_normal((b, NQ)).astype(np.float16)
    w = np.ones(HD, np.float16)
    cos, sin = O.rope_table(512)
    kin = k.copy()
    ctx = O.decode_layer(q, kin, v, gate, w, w, cos, sin, lens, lens + 1,
                         O.ptr_table(ks), O.ptr_table(vs))
    for i in range(b):
        assert np.array_equal(vs[i][lens[i]].view(np.uint16), v[i].view(np.uint16))
        assert np.array_equal(ks[i][lens[i]].view(np.uint16), kin[i].view(np.uint16))
    assert np.isfinite(ctx.astype(np.float32)).all()
