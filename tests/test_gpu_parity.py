"""GPU parity: liboxi_kv (through the C ABI) against the CPU oracle and against the
reference's own kernels on the same GPU (fixture `ref` of tests/conftest.py: tests that use it are
skipped, not passed, where the prebuilt cubins are missing).

Bars: K/V/q/conv-state bytes bit-exact vs the reference kernels (K and q within
one f16 ulp vs the CPU oracle, whose rsqrt is correctly rounded); attention
output max-abs <= 2e-3 (fp16 storage, fp32 accumulate)."""
import numpy as np
import pytest
import torch

from tests.kvcase import NQ, NKV, HD, HIDDEN, DecodeCase, dev_ptr_table, u32, ulp_diff_f16

pytestmark = pytest.mark.gpu

ATTN_TOL = 2e-3


@pytest.fixture(scope="module")
def kv():
    from oxide_infer_b200 import KvPath, build
    build.build()
    p = KvPath(0, max_batch=256, max_seq_len=40960, max_prefill_rows=1024)
    yield p
    assert p.device_status() == 0
    p.close()


@pytest.fixture(scope="module")
def O():
    from oracle import cpu
    cpu.build()
    return cpu


def _np(t):
    return t.detach().cpu().numpy()


def _bits(a):
    return np.ascontiguousarray(a).view(np.uint16)


# ------------------------------------------------------------------ append --

def _run_append(kv, case):
    d = case.device()
    kv.append(d.q, d.k, d.v, d.q_norm_w, d.k_norm_w, d.cos, d.sin, d.pos_ids, d.k_ptrs, d.v_ptrs)
    torch.cuda.synchronize()
    return d


def _oracle_append(O, case):
    h = case.host()
    O.qk_rmsnorm(h.q, case.q_norm_w)
    O.qk_rmsnorm(h.k, case.k_norm_w)
    O.rope(h.q, case.cos, case.sin, case.pos_ids)
    O.rope(h.k, case.cos, case.sin, case.pos_ids)
    O.kv_copy(h.k_ptrs, h.k, case.pos_ids)
    O.kv_copy(h.v_ptrs, h.v, case.pos_ids)
    return h


@pytest.mark.parametrize("seed,partial,theta", [(0, 0.5, 1e6), (1, 1.0, 1e4)])
def test_append_vs_oracle(kv, O, seed, partial, theta):
    lens = np.random.default_rng(seed).integers(64, 513, 8)
    case = DecodeCase(lens, seed=seed, theta=theta, partial=partial)
    d = _run_append(kv, case)
    h = _oracle_append(O, case)
    for i, n in enumerate(case.lens):
        kd, vd = _np(d.k_cache[i]), _np(d.v_cache[i])
        # V: pure copy, bit-exact; untouched rows stay untouched
        assert np.array_equal(_bits(vd), _bits(h.v_cache[i]))
        assert np.array_equal(_bits(kd[:n]), _bits(case.k_cache[i][:n]))
        ulp = ulp_diff_f16(kd[n], h.k_cache[i][n])
        assert ulp.max() <= 1, ulp.max()
    ulp_q = ulp_diff_f16(_np(d.q), h.q)
    assert ulp_q.max() <= 1
    assert (ulp_q != 0).mean() < 0.02  # rsqrt.approx vs correctly rounded: rare last-bit flips


@pytest.mark.parametrize("seed,partial,theta,b", [(0, 0.5, 1e6, 8), (1, 1.0, 1e4, 8), (2, 0.5, 1e6, 128)])
def test_append_bit_exact_vs_reference_kernels(kv, ref, seed, partial, theta, b):
    if ref is None:
        pytest.skip("oracle/_ref cubins not built")
    lens = np.random.default_rng(seed).integers(64, 513, b)
    case = DecodeCase(lens, seed=seed, theta=theta, partial=partial)
    d = _run_append(kv, case)
    r = case.device()
    ref.append(r.q, r.k, r.v, r.q_norm_w, r.k_norm_w, r.cos, r.sin, r.pos_ids, r.k_ptrs, r.v_ptrs, b)
    torch.cuda.synchronize()
    assert torch.equal(d.q.view(torch.int16), r.q.view(torch.int16))
    for i in range(b):
        assert torch.equal(d.k_cache[i].view(torch.int16), r.k_cache[i].view(torch.int16))
        assert torch.equal(d.v_cache[i].view(torch.int16), r.v_cache[i].view(torch.int16))


def test_unfused_operators_match_reference_kernels(kv, ref, O):
    case = DecodeCase([70, 129, 300, 511], seed=5)
    d = case.device()
    kv.qk_rmsnorm(d.q, d.q_norm_w)
    kv.qk_rmsnorm(d.k, d.k_norm_w)
    kv.rope(d.q, d.cos, d.sin, d.pos_ids)
    kv.rope(d.k, d.cos, d.sin, d.pos_ids)
    kv.kv_copy(d.k_ptrs, d.k, d.pos_ids)
    kv.kv_copy(d.v_ptrs, d.v, d.pos_ids)
    f = _run_append(kv, case)  # the fused kernel must equal the unfused sequence bit for bit
    torch.cuda.synchronize()
    assert torch.equal(d.q.view(torch.int16), f.q.view(torch.int16))
    for i in range(case.b):
        assert torch.equal(d.k_cache[i].view(torch.int16), f.k_cache[i].view(torch.int16))
        assert torch.equal(d.v_cache[i].view(torch.int16), f.v_cache[i].view(torch.int16))
    # sigmoid gate vs oracle (and reference kernel when present)
    ctx = torch.randn(4, NQ, HD, device="cuda").half()
    mine = ctx.clone()
    kv.sigmoid_gate(mine, d.gate)
    want = _np(ctx).copy()
    O.sigmoid_gate(want, case.gate)
    torch.cuda.synchronize()
    assert ulp_diff_f16(_np(mine), want).max() <= 1
    if ref is not None:
        theirs = ctx.clone()
        ref.sigmoid_gate(theirs, d.gate, 4)
        torch.cuda.synchronize()
        assert torch.equal(mine.view(torch.int16), theirs.view(torch.int16))


# ---------------------------------------------------------- decode attention --

def _decode_all(kv, ref, O, case, window, use_gate=True):
    """Append + gated decode attention on every side; returns dict of ctx arrays (float32)."""
    out = {}
    d = _run_append(kv, case)
    kv.decode_attn(d.ctx, d.q, d.gate if use_gate else None, d.k_ptrs, d.v_ptrs, d.seq_lens, window)
    torch.cuda.synchronize()
    out["oxi"] = _np(d.ctx).astype(np.float32)
    h = _oracle_append(O, case)
    out["oracle"] = O.decode_attn(h.q, case.gate if use_gate else None, h.k_ptrs, h.v_ptrs,
                                  case.seq_lens, window).astype(np.float32)
    if ref is not None:
        r = case.device()
        ref.append(r.q, r.k, r.v, r.q_norm_w, r.k_norm_w, r.cos, r.sin, r.pos_ids, r.k_ptrs,
                   r.v_ptrs, case.b)
        ref.decode_attention(r.ctx, r.q, r.gate if use_gate else None, r.k_ptrs, r.v_ptrs,
                             r.seq_lens, case.b, window, int(case.seq_lens.max()))
        torch.cuda.synchronize()
        out["ref"] = _np(r.ctx).astype(np.float32)
    return out


@pytest.mark.parametrize("window", [0, 256])
def test_decode_config1(kv, ref, O, window):
    """Config 1: batch 8, context uniform 64..512, seed 0; append then gated attention."""
    lens = np.random.default_rng(0).integers(64, 513, 8)
    case = DecodeCase(lens, seed=0)
    out = _decode_all(kv, ref, O, case, window)
    assert np.abs(out["oxi"] - out["oracle"]).max() <= ATTN_TOL
    if "ref" in out:
        assert np.abs(out["oxi"] - out["ref"]).max() <= ATTN_TOL
        assert np.abs(out["ref"] - out["oracle"]).max() <= ATTN_TOL  # the oracle tracks the reference


@pytest.mark.parametrize("lens", [[1], [0, 1, 2], [31, 32, 33], [255, 256, 257, 511, 512, 513],
                                  [1023, 1024, 1025], [4095]])
@pytest.mark.parametrize("window", [0, 256])
def test_decode_edges(kv, ref, O, lens, window):
    """Lengths around every stage (32), work-item (256) and reference chunk (128) boundary.
    `lens` are old lengths: a 0 means the appended token is the only key."""
    case = DecodeCase(lens, seed=len(lens) + window)
    out = _decode_all(kv, ref, O, case, window)
    assert np.isfinite(out["oxi"]).all()
    assert np.abs(out["oxi"] - out["oracle"]).max() <= ATTN_TOL
    if "ref" in out:
        assert np.abs(out["oxi"] - out["ref"]).max() <= ATTN_TOL


def test_decode_no_gate_and_large_scores(kv, ref, O):
    case = DecodeCase([300, 700], seed=9, kscale=3.0)  # peaked softmax
    out = _decode_all(kv, ref, O, case, 0, use_gate=False)
    assert np.abs(out["oxi"] - out["oracle"]).max() <= ATTN_TOL


def test_decode_ragged_batch128(kv, ref, O):
    """Config 2 shape, one layer: batch 128, context uniform 1024..4096."""
    lens = np.random.default_rng(2).integers(1024, 4097, 128) - 1
    case = DecodeCase(lens, seed=2)
    d = _run_append(kv, case)
    kv.decode_attn(d.ctx, d.q, d.gate, d.k_ptrs, d.v_ptrs, d.seq_lens, 0)
    torch.cuda.synchronize()
    mine = _np(d.ctx).astype(np.float32)
    if ref is not None:
        r = case.device()
        ref.append(r.q, r.k, r.v, r.q_norm_w, r.k_norm_w, r.cos, r.sin, r.pos_ids, r.k_ptrs, r.v_ptrs, 128)
        ref.decode_attention(r.ctx, r.q, r.gate, r.k_ptrs, r.v_ptrs, r.seq_lens, 128, 0,
                             int(case.seq_lens.max()))
        torch.cuda.synchronize()
        assert np.abs(mine - _np(r.ctx).astype(np.float32)).max() <= ATTN_TOL
    # oracle on a subset of rows (CPU time), through the same tables
    rows = [0, 17, 63, 127]
    h = _oracle_append(O, case)
    ctx = O.decode_attn(np.ascontiguousarray(h.q[rows]), np.ascontiguousarray(case.gate[rows]),
                        np.ascontiguousarray(h.k_ptrs[rows]), np.ascontiguousarray(h.v_ptrs[rows]),
                        np.ascontiguousarray(case.seq_lens[rows]), 0).astype(np.float32)
    assert np.abs(mine[rows] - ctx).max() <= ATTN_TOL


def test_decode_batch_composition_invariance(kv):
    """A row's output bytes do not depend on which rows share the launch."""
    lens = np.random.default_rng(3).integers(100, 3000, 32)
    case = DecodeCase(lens, seed=3)
    d = _run_append(kv, case)
    kv.decode_attn(d.ctx, d.q, d.gate, d.k_ptrs, d.v_ptrs, d.seq_lens, 0)
    full = d.ctx.clone()
    for i in (0, 13, 31):
        one = torch.zeros(1, NQ, HD, dtype=torch.float16, device="cuda")
        kv.decode_attn(one, d.q[i:i + 1].contiguous(), d.gate[i:i + 1].contiguous(),
                       d.k_ptrs[i:i + 1].contiguous(), d.v_ptrs[i:i + 1].contiguous(),
                       d.seq_lens[i:i + 1].contiguous(), 0)
        torch.cuda.synchronize()
        assert torch.equal(one[0].view(torch.int16), full[i].view(torch.int16))
    # and repeated launches are deterministic
    again = torch.zeros_like(full)
    kv.decode_attn(again, d.q, d.gate, d.k_ptrs, d.v_ptrs, d.seq_lens, 0)
    torch.cuda.synchronize()
    assert torch.equal(again.view(torch.int16), full.view(torch.int16))


def test_decode_long_rows_merge_by_slices_independent_of_launch_shape(kv):
    """Rows of more than 16 key ranges are merged in slices by several CTAs; how many CTAs share a
    row depends on the batch and on the handle, the bytes must not: a long row alone, among many
    short rows (fewer CTAs per row) and through a handle with another maximum length."""
    from oxide_infer_b200 import KvPath
    lens = np.concatenate([[20000, 4097, 33000, 8191], np.random.default_rng(5).integers(10, 600, 250)])  # 254 rows: 2 CTAs per row here, 8 below
    case = DecodeCase(lens, seed=5)
    d = _run_append(kv, case)
    kv.decode_attn(d.ctx, d.q, d.gate, d.k_ptrs, d.v_ptrs, d.seq_lens, 0)
    full = d.ctx.clone()
    sub = lambda t, i, n: t[i:i + n].contiguous()
    other = KvPath(0, max_batch=4, max_seq_len=131072, max_prefill_rows=0)
    for h in (kv, other):
        for i, n in ((0, 1), (2, 1), (0, 4), (1, 3)):
            out = torch.zeros(n, NQ, HD, dtype=torch.float16, device="cuda")
            h.decode_attn(out, sub(d.q, i, n), sub(d.gate, i, n), sub(d.k_ptrs, i, n), sub(d.v_ptrs, i, n),
                          sub(d.seq_lens, i, n), 0)
            torch.cuda.synchronize()
            assert torch.equal(out.view(torch.int16), full[i:i + n].view(torch.int16))
    # windows cut a long row back to one slice or to a few
    for window in (4096, 5000):
        a = torch.zeros_like(full)
        kv.decode_attn(a, d.q, d.gate, d.k_ptrs, d.v_ptrs, d.seq_lens, window)
        one = torch.zeros(1, NQ, HD, dtype=torch.float16, device="cuda")
        kv.decode_attn(one, sub(d.q, 2, 1), sub(d.gate, 2, 1), sub(d.k_ptrs, 2, 1), sub(d.v_ptrs, 2, 1),
                       sub(d.seq_lens, 2, 1), window)
        torch.cuda.synchronize()
        assert torch.equal(one[0].view(torch.int16), a[2].view(torch.int16))
    assert kv.device_status() == 0 and other.device_status() == 0


def test_reference_known_answer_cases_on_gpu(kv, O):
    """The reference's own test shapes through the library: uniform-softmax mean position
    (debug_online_attn.rs), pat()-seeded rows 300/180/64/300 vs f64 < 3e-3
    (test_split_attention.rs), window set of test_swa_attention.rs < 2e-3."""
    seq = 300
    q = torch.ones(1, NQ, HD, dtype=torch.float16, device="cuda")
    k = torch.ones(seq, NKV, HD, dtype=torch.float16, device="cuda")
    v = torch.arange(seq, dtype=torch.float16, device="cuda")[:, None, None].expand(seq, NKV, HD).contiguous()
    ctx = torch.zeros(1, NQ, HD, dtype=torch.float16, device="cuda")
    sl = u32(np.array([seq], np.uint32))
    for window, want in [(0, 149.5), (256, 171.5)]:
        kv.decode_attn(ctx, q, None, dev_ptr_table([k]), dev_ptr_table([v]), sl, window)
        torch.cuda.synchronize()
        # v values up to 299 carry f16 steps of 0.125..0.25 and weights are f16 on the PV path
        assert (ctx.float() - want).abs().max().item() <= 0.13
    rows = [300, 180, 64, 300]
    qf = O.pat(1, 4 * NQ * HD).reshape(4, NQ, HD)
    ks = [O.pat(2 + r, 300 * NKV * HD, 2.0) for r in range(4)]
    vs = [O.pat(9 + r, 300 * NKV * HD) for r in range(4)]
    dq = torch.from_numpy(O.f2h(qf)).cuda()
    dk = [torch.from_numpy(O.f2h(a)).cuda() for a in ks]
    dv = [torch.from_numpy(O.f2h(a)).cuda() for a in vs]
    ctx = torch.zeros(4, NQ, HD, dtype=torch.float16, device="cuda")
    for window in (0, 256):
        kv.decode_attn(ctx, dq, None, dev_ptr_table(dk), dev_ptr_table(dv), u32(np.array(rows, np.uint32)), window)
        torch.cuda.synchronize()
        for r, slen in enumerate(rows):
            want = O.attention_f64(qf[r], ks[r], vs[r], slen, window)
            assert np.abs(_np(ctx[r]).astype(np.float64) - want).max() < 3e-3
    for window in (0, 512, 300, 257, 256, 128):
        kv.decode_attn(ctx[:1], dq[:1].contiguous(), None, dev_ptr_table(dk[:1]), dev_ptr_table(dv[:1]),
                       u32(np.array([300], np.uint32)), window)
        torch.cuda.synchronize()
        want = O.attention_f64(qf[0], ks[0], vs[0], 300, window)
        assert np.abs(_np(ctx[0]).astype(np.float64) - want).max() < 2e-3


def test_misaligned_pointer_is_reported_not_dereferenced(kv):
    case = DecodeCase([40, 50], seed=4)
    d = case.device()
    bad = d.k_ptrs.clone()
    bad[1] += 2
    before = d.ctx.clone()
    kv.decode_attn(d.ctx, d.q, d.gate, bad, d.v_ptrs, d.seq_lens, 0)
    assert kv.device_status() & 1
    assert torch.equal(d.ctx[1], before[1])      # the bad row is skipped
    assert d.ctx[0].abs().sum().item() > 0        # the good row is computed
    assert kv.device_status() == 0               # the word is cleared by reading it


def test_host_side_argument_errors(kv):
    from oxide_infer_b200 import OxiError
    case = DecodeCase([10], seed=1)
    d = case.device()
    with pytest.raises(OxiError) as e:
        kv.decode_attn(d.ctx, d.q, d.gate, None, d.v_ptrs, d.seq_lens, 0)
    assert e.value.code == -1
    with pytest.raises(OxiError) as e:
        kv.decode_attn(d.ctx, d.q, d.gate, d.k_ptrs, d.v_ptrs, d.seq_lens, 0, batch=0)
    assert e.value.code == -2
    with pytest.raises(OxiError) as e:
        kv.decode_attn(d.ctx, d.q, d.gate, d.k_ptrs, d.v_ptrs, d.seq_lens, 0, batch=100000)
    assert e.value.code == -2
    with pytest.raises(OxiError) as e:
        kv.prefill_attn(d.ctx, d.q, d.gate, d.k_ptrs, d.v_ptrs, d.seq_lens, 0, rows=10 ** 6)
    assert e.value.code == -2


# -------------------------------------------------------------------- conv --

def _conv_inputs(b, seed):
    rng = np.random.default_rng(seed)
    state = [rng.standard_normal((HIDDEN, 6), dtype=np.float32).astype(np.float16) for _ in range(b)]
    bcx = rng.standard_normal((b, 3 * HIDDEN), dtype=np.float32).astype(np.float16)
    w = (rng.standard_normal((HIDDEN, 7), dtype=np.float32) * 0.1).astype(np.float16)
    return state, bcx, w


@pytest.mark.parametrize("b", [1, 7, 128])
def test_conv_decode_bit_exact(kv, ref, O, b):
    state, bcx, w = _conv_inputs(b, b)
    hs = [s.copy() for s in state]
    y_want = O.conv_decode(O.ptr_table(hs), bcx, w)
    ds = [torch.from_numpy(s.copy()).cuda() for s in state]
    dbcx, dw = torch.from_numpy(bcx).cuda(), torch.from_numpy(w).cuda()
    y = torch.zeros(b, HIDDEN, dtype=torch.float16, device="cuda")
    kv.conv_decode(y, dev_ptr_table(ds), dbcx, dw)
    torch.cuda.synchronize()
    assert np.array_equal(_bits(_np(y)), _bits(y_want))
    for a, h in zip(ds, hs):
        assert np.array_equal(_bits(_np(a)), _bits(h))
    if ref is not None:
        rs = [torch.from_numpy(s.copy()).cuda() for s in state]
        yr = torch.zeros_like(y)
        ref.conv_decode(yr, dev_ptr_table(rs), dbcx, dw, b)
        torch.cuda.synchronize()
        assert torch.equal(y.view(torch.int16), yr.view(torch.int16))
        for a, r in zip(ds, rs):
            assert torch.equal(a.view(torch.int16), r.view(torch.int16))


def test_conv_unit_weights_zero_state_gpu(kv):
    """kernels/src/conv.rs:224-268 on the pointer-table kernel: every output == 2.0."""
    st = [torch.zeros(HIDDEN, 6, dtype=torch.float16, device="cuda")]
    bcx = torch.ones(1, 3 * HIDDEN, dtype=torch.float16, device="cuda")
    bcx[:, 2 * HIDDEN:] = 2.0
    w = torch.ones(HIDDEN, 7, dtype=torch.float16, device="cuda")
    y = torch.zeros(1, HIDDEN, dtype=torch.float16, device="cuda")
    kv.conv_decode(y, dev_ptr_table(st), bcx, w)
    torch.cuda.synchronize()
    assert (y == 2.0).all() and (st[0][:, 5] == 2.0).all() and (st[0][:, :5] == 0).all()


@pytest.mark.parametrize("lens", [[1, 5, 6, 7, 19], [128, 128], [3], [16, 16, 1, 15, 17, 33], [13, 40, 2, 9], [250, 1, 5],
                                  [10, 6, 16, 31, 1, 1, 1, 64]])
def test_conv_prefill_bit_exact(kv, ref, O, lens):
    rng = np.random.default_rng(sum(lens))
    rows = sum(lens)
    bcx = rng.standard_normal((rows, 3 * HIDDEN), dtype=np.float32).astype(np.float16)
    w = (rng.standard_normal((HIDDEN, 7), dtype=np.float32) * 0.1).astype(np.float16)
    carry0 = [rng.standard_normal((HIDDEN, 6), dtype=np.float32).astype(np.float16) for _ in lens]
    origin, lpos, owner = [], [], []
    r0 = 0
    for i, n in enumerate(lens):
        origin += [r0] * n
        lpos += list(range(n))
        owner += [i] * n
        r0 += n
    origin, lpos = np.array(origin, np.uint32), np.array(lpos, np.uint32)
    hc = [c.copy() for c in carry0]
    y_want = O.conv_prefill_wave(O.ptr_table([hc[i] for i in owner]), origin, lpos, bcx, w)
    dc = [torch.from_numpy(c.copy()).cuda() for c in carry0]
    y = torch.zeros(rows, HIDDEN, dtype=torch.float16, device="cuda")
    dbcx, dw = torch.from_numpy(bcx).cuda(), torch.from_numpy(w).cuda()
    kv.conv_prefill(y, dev_ptr_table([dc[i] for i in owner]), u32(origin), u32(lpos), dbcx, dw)
    torch.cuda.synchronize()
    assert np.array_equal(_bits(_np(y)), _bits(y_want))
    for a, h in zip(dc, hc):
        assert np.array_equal(_bits(_np(a)), _bits(h))
    if ref is not None:
        rc = [torch.from_numpy(c.copy()).cuda() for c in carry0]
        yr = torch.zeros_like(y)
        pool = torch.zeros(rows, HIDDEN, 6, dtype=torch.float16, device="cuda")
        ref.conv_prefill_wave(yr, pool, dev_ptr_table([rc[i] for i in owner]), u32(origin), u32(lpos),
                              dbcx, dw, rows, [rc[i] for i in owner], origin)
        torch.cuda.synchronize()
        assert torch.equal(y.view(torch.int16), yr.view(torch.int16))
        for a, r in zip(dc, rc):
            assert torch.equal(a.view(torch.int16), r.view(torch.int16))


def test_conv_prefill_chunking_invariance_and_decode_equivalence(kv):
    """A prompt's conv outputs and final state do not depend on how it is cut into chunks: 300 rows as one
    chunk, as waves of 128 + 128 + 44 rows carried through the persistent state, as 7 + 293, and token by
    token through the decode kernel - all bit-identical."""
    rng = np.random.default_rng(300)
    n = 300
    bcx = torch.from_numpy(rng.standard_normal((n, 3 * HIDDEN), dtype=np.float32).astype(np.float16)).cuda()
    w = torch.from_numpy((rng.standard_normal((HIDDEN, 7), dtype=np.float32) * 0.1).astype(np.float16)).cuda()
    state0 = torch.from_numpy(rng.standard_normal((HIDDEN, 6), dtype=np.float32).astype(np.float16)).cuda()

    def run(cuts):
        st = state0.clone()
        y = torch.zeros(n, HIDDEN, dtype=torch.float16, device="cuda")
        lo = 0
        for m in cuts:
            kv.conv_prefill(y[lo:lo + m], dev_ptr_table([st] * m), u32(np.zeros(m, np.uint32)),
                            u32(np.arange(m, dtype=np.uint32)), bcx[lo:lo + m].contiguous(), w)
            lo += m
        torch.cuda.synchronize()
        assert lo == n
        return y, st

    y1, s1 = run([300])
    for cuts in ([128, 128, 44], [7, 293], [1] * 5 + [295]):
        y2, s2 = run(cuts)
        assert torch.equal(y1.view(torch.int16), y2.view(torch.int16))
        assert torch.equal(s1.view(torch.int16), s2.view(torch.int16))
    st = state0.clone()
    yd = torch.zeros(n, HIDDEN, dtype=torch.float16, device="cuda")
    ptr = dev_ptr_table([st])
    for t in range(n):
        kv.conv_decode(yd[t:t + 1], ptr, bcx[t:t + 1].contiguous(), w)
    torch.cuda.synchronize()
    assert torch.equal(y1.view(torch.int16), yd.view(torch.int16))
    assert torch.equal(s1.view(torch.int16), st.view(torch.int16))


# ----------------------------------------------------------------- prefill --

def _prefill_case(chunks, cache_len, seed, kscale=1.0):
    """chunks: list of (rows, p0).  Each chunk is one request with its own cache holding
    positions [0, p0+rows).  Returns numpy q, gate, caches, per-row tables."""
    rng = np.random.default_rng(seed)
    total = sum(c[0] for c in chunks)
    f16 = lambda *s, sc=1.0: (rng.standard_normal(s, dtype=np.float32) * sc).astype(np.float16)
    q, gate = f16(total, NQ, HD), f16(total, NQ)
    ks = [f16(max(cache_len, p0 + n), NKV, HD, sc=kscale) for n, p0 in chunks]
    vs = [f16(max(cache_len, p0 + n), NKV, HD) for n, p0 in chunks]
    owner, slen = [], []
    for i, (n, p0) in enumerate(chunks):
        owner += [i] * n
        slen += [p0 + r + 1 for r in range(n)]
    return q, gate, ks, vs, owner, np.array(slen, np.uint32)


@pytest.mark.parametrize("window", [0, 256])
@pytest.mark.parametrize("chunks", [[(96, 0), (128, 400)], [(5, 0), (1, 77), (30, 3), (64, 1000)],
                                    [(128, 4000)]])
def test_prefill_attn(kv, ref, O, chunks, window):
    """Chunk shapes of test_gemm_attention.rs ({96 rows @0, 128 rows @400}) plus ragged waves;
    compared with the online kernel + gate per row (the reference's own cross-check)."""
    q, gate, ks, vs, owner, slen = _prefill_case(chunks, 600, seed=len(chunks) + window)
    rows = len(owner)
    dk = [torch.from_numpy(a).cuda() for a in ks]
    dv = [torch.from_numpy(a).cuda() for a in vs]
    dq, dg = torch.from_numpy(q).cuda(), torch.from_numpy(gate).cuda()
    kp, vp = dev_ptr_table([dk[i] for i in owner]), dev_ptr_table([dv[i] for i in owner])
    ctx = torch.zeros(rows, NQ, HD, dtype=torch.float16, device="cuda")
    kv.prefill_attn(ctx, dq, dg, kp, vp, u32(slen), window)
    torch.cuda.synchronize()
    mine = _np(ctx).astype(np.float32)
    hk, hv = O.ptr_table([ks[i] for i in owner]), O.ptr_table([vs[i] for i in owner])
    want = O.attn_online(q, hk, hv, slen, window)
    O.sigmoid_gate(want, gate)
    assert np.abs(mine - want.astype(np.float32)).max() <= ATTN_TOL
    if ref is not None:
        rctx = torch.zeros_like(ctx)
        ref.attn_online(rctx, dq, kp, vp, u32(slen), rows, window)
        ref.sigmoid_gate(rctx, dg, rows)
        torch.cuda.synchronize()
        assert np.abs(mine - _np(rctx).astype(np.float32)).max() <= ATTN_TOL


def test_prefill_full_size_wave_against_reference_and_request_order(ref):
    """Configuration 4 at full size (32 requests x 128 new rows, prefixes U[0, 8192], 4096 wave rows): every
    row against the reference's own online kernel + gate kernel, and a size-independent property: the order
    of the requests inside the wave must not change any request's output bytes."""
    from oxide_infer_b200 import KvPath
    nseq, new = 32, 128
    rows = nseq * new
    rng = np.random.default_rng(4)
    prefix = rng.integers(0, 8193, nseq)
    kvp = KvPath(0, max_batch=8, max_seq_len=8192 + new, max_prefill_rows=rows)
    g = torch.Generator(device="cuda").manual_seed(44)
    rn = lambda *s: torch.empty(*s, dtype=torch.float16, device="cuda").normal_(generator=g)
    kc = [rn(int(p) + new, NKV, HD) for p in prefix]
    vc = [rn(int(p) + new, NKV, HD) for p in prefix]
    q, gate = rn(rows, NQ, HD), rn(rows, NQ)

    def run(order):
        owner = np.repeat(order, new)
        lens = (prefix[owner] + np.tile(np.arange(new), nseq) + 1).astype(np.int32)
        kp = torch.tensor([kc[i].data_ptr() for i in owner], dtype=torch.int64, device="cuda")
        vp = torch.tensor([vc[i].data_ptr() for i in owner], dtype=torch.int64, device="cuda")
        src = torch.from_numpy(np.concatenate([np.arange(i * new, (i + 1) * new) for i in order])).cuda()
        qq, gg = q[src].contiguous(), gate[src].contiguous()  # request i keeps its q and gate rows
        ctx = torch.zeros(rows, NQ, HD, dtype=torch.float16, device="cuda")
        dl = torch.from_numpy(lens).cuda()
        kvp.prefill_attn(ctx, qq, gg, kp, vp, dl, 0)
        torch.cuda.synchronize()
        return ctx, (qq, gg, kp, vp, dl), src

    base, args, _ = run(np.arange(nseq))
    assert kvp.device_status() == 0 and torch.isfinite(base.float()).all()
    perm = np.random.default_rng(9).permutation(nseq)
    other, _, src = run(perm)
    assert torch.equal(other.view(torch.int16), base[src].view(torch.int16))
    if ref is not None:
        qq, gg, kp, vp, dl = args
        rctx = torch.zeros_like(base)
        ref.attn_online(rctx, qq, kp, vp, dl, rows, 0)
        ref.sigmoid_gate(rctx, gg, rows)
        torch.cuda.synchronize()
        assert (base.float() - rctx.float()).abs().max().item() <= ATTN_TOL


def test_prefill_wave_of_more_than_1024_blocks(O):
    """Waves beyond 65,536 rows (1024 blocks of 64) are ordered by the general counting-sort plan kernel: the
    bytes must equal those of the same requests sent as two smaller waves (ranked by the small plan kernel),
    and sampled requests must match the oracle."""
    from oxide_infer_b200 import KvPath
    nseq, new = 1040, 64  # 1040 blocks
    rows = nseq * new
    rng = np.random.default_rng(12)
    prefix = rng.integers(0, 300, nseq)
    kvp = KvPath(0, max_batch=8, max_seq_len=512, max_prefill_rows=rows)
    g = torch.Generator(device="cuda").manual_seed(12)
    rn = lambda *s: torch.empty(*s, dtype=torch.float16, device="cuda").normal_(generator=g)
    cap = prefix + new
    offs = np.concatenate([[0], np.cumsum(cap)])
    kslab, vslab = rn(int(offs[-1]), NKV, HD), rn(int(offs[-1]), NKV, HD)
    q, gate = rn(rows, NQ, HD), rn(rows, NQ)
    owner = np.repeat(np.arange(nseq), new)
    lens = (prefix[owner] + np.tile(np.arange(new), nseq) + 1).astype(np.int32)
    kp = torch.from_numpy(kslab.data_ptr() + offs[owner] * 1024).cuda()
    vp = torch.from_numpy(vslab.data_ptr() + offs[owner] * 1024).cuda()
    dl = torch.from_numpy(lens).cuda()
    ctx = torch.zeros(rows, NQ, HD, dtype=torch.float16, device="cuda")
    kvp.prefill_attn(ctx, q, gate, kp, vp, dl, 0)
    torch.cuda.synchronize()
    assert kvp.device_status() == 0
    two = torch.zeros_like(ctx)
    half = (nseq // 2) * new
    for lo, hi in ((0, half), (half, rows)):
        kvp.prefill_attn(two[lo:hi], q[lo:hi], gate[lo:hi], kp[lo:hi].contiguous(), vp[lo:hi].contiguous(),
                         dl[lo:hi].contiguous(), 0)
    torch.cuda.synchronize()
    assert torch.equal(ctx.view(torch.int16), two.view(torch.int16))
    hk, hv = kslab.cpu().numpy(), vslab.cpu().numpy()
    for i in (0, 517, nseq - 1):
        sl = slice(i * new, (i + 1) * new)
        kc, vc = hk[offs[i]:offs[i + 1]], hv[offs[i]:offs[i + 1]]
        want = O.attn_online(q[sl].cpu().numpy(), O.ptr_table([kc] * new), O.ptr_table([vc] * new),
                             lens[sl].astype(np.uint32), 0)
        O.sigmoid_gate(want, gate[sl].cpu().numpy())
        assert np.abs(ctx[sl].float().cpu().numpy() - want.astype(np.float32)).max() <= ATTN_TOL


def test_prefill_attn_many_runs_per_block(kv, O):
    """Run boundaries at every row: 70 single-row chunks of 70 requests (64 runs in the first block), then
    two caches alternating row by row (equal pointers that are not neighbours must not merge), with
    skipped rows (length 0) at the block's and the warp's edges."""
    rng = np.random.default_rng(77)
    chunks = [(1, int(p)) for p in rng.integers(0, 200, 70)]
    q, gate, ks, vs, owner, slen = _prefill_case(chunks, 1, seed=77)
    for case in range(2):
        if case == 1:  # rows alternate between cache 0 and cache 1, lengths grow row by row
            owner = [r & 1 for r in range(70)]
            ks = [rng.standard_normal((300, NKV, HD), dtype=np.float32).astype(np.float16) for _ in (0, 1)]
            vs = [rng.standard_normal((300, NKV, HD), dtype=np.float32).astype(np.float16) for _ in (0, 1)]
            slen = np.array([100 + 2 * r for r in range(70)], np.uint32)
            slen[[0, 31, 32, 63, 64]] = 0
        rows = len(owner)
        dk = [torch.from_numpy(a).cuda() for a in ks]
        dv = [torch.from_numpy(a).cuda() for a in vs]
        dq, dg = torch.from_numpy(q).cuda(), torch.from_numpy(gate).cuda()
        kp, vp = dev_ptr_table([dk[i] for i in owner]), dev_ptr_table([dv[i] for i in owner])
        ctx = torch.full((rows, NQ, HD), 5.0, dtype=torch.float16, device="cuda")
        kv.prefill_attn(ctx, dq, dg, kp, vp, u32(slen), 0)
        torch.cuda.synchronize()
        status = kv.device_status()
        mine = _np(ctx).astype(np.float32)
        live = slen != 0
        assert status == (0 if live.all() else 2)  # OXI_DEV_BAD_SEQ_LEN for the skipped rows
        hk, hv = O.ptr_table([ks[i] for i in owner]), O.ptr_table([vs[i] for i in owner])
        want = O.attn_online(q, hk, hv, np.where(live, slen, 1).astype(np.uint32), 0)
        O.sigmoid_gate(want, gate)
        assert np.abs(mine[live] - want.astype(np.float32)[live]).max() <= ATTN_TOL
        assert (mine[~live] == 5.0).all()  # skipped rows are not written


# ------------------------------------------------- fused append + decode --

@pytest.mark.parametrize("lens,window", [([64, 100, 511, 300, 77, 256, 255, 129], 0),
                                         ([0, 1, 2, 31, 32, 33], 0), ([255, 256, 257, 511, 512, 513], 256),
                                         ([1023, 1024, 1025, 4095], 0), ([300, 700, 5], 128)])
def test_fused_append_decode_matches_unfused_bitwise(kv, lens, window):
    """oxi_append_decode (RMSNorm + RoPE + KV append inside the attention kernel) must leave the
    same cache bytes and the same context bytes as oxi_append followed by oxi_decode_attn, and
    must not modify q."""
    case = DecodeCase(lens, seed=31 + len(lens) + window)
    a, f = case.device(), case.device()
    kv.append(a.q, a.k, a.v, a.q_norm_w, a.k_norm_w, a.cos, a.sin, a.pos_ids, a.k_ptrs, a.v_ptrs)
    kv.decode_attn(a.ctx, a.q, a.gate, a.k_ptrs, a.v_ptrs, a.seq_lens, window)
    q_before = f.q.clone()
    kv.append_decode(f.ctx, f.q, f.k, f.v, f.gate, f.q_norm_w, f.k_norm_w, f.cos, f.sin, f.pos_ids, f.seq_lens,
                     f.k_ptrs, f.v_ptrs, window)
    torch.cuda.synchronize()
    assert torch.equal(a.ctx.view(torch.int16), f.ctx.view(torch.int16))
    assert torch.equal(f.q.view(torch.int16), q_before.view(torch.int16))
    for i in range(case.b):
        assert torch.equal(a.k_cache[i].view(torch.int16), f.k_cache[i].view(torch.int16))
        assert torch.equal(a.v_cache[i].view(torch.int16), f.v_cache[i].view(torch.int16))


def test_fused_append_decode_ragged_batch128(kv, ref):
    lens = np.random.default_rng(7).integers(1024, 4097, 128) - 1
    case = DecodeCase(lens, seed=7)
    f = case.device()
    kv.append_decode(f.ctx, f.q, f.k, f.v, f.gate, f.q_norm_w, f.k_norm_w, f.cos, f.sin, f.pos_ids, f.seq_lens,
                     f.k_ptrs, f.v_ptrs, 0)
    a = case.device()
    kv.append(a.q, a.k, a.v, a.q_norm_w, a.k_norm_w, a.cos, a.sin, a.pos_ids, a.k_ptrs, a.v_ptrs)
    kv.decode_attn(a.ctx, a.q, a.gate, a.k_ptrs, a.v_ptrs, a.seq_lens, 0)
    torch.cuda.synchronize()
    assert torch.equal(a.ctx.view(torch.int16), f.ctx.view(torch.int16))
    if ref is not None:
        r = case.device()
        ref.append(r.q, r.k, r.v, r.q_norm_w, r.k_norm_w, r.cos, r.sin, r.pos_ids, r.k_ptrs, r.v_ptrs, 128)
        ref.decode_attention(r.ctx, r.q, r.gate, r.k_ptrs, r.v_ptrs, r.seq_lens, 128, 0, int(case.seq_lens.max()))
        torch.cuda.synchronize()
        assert np.abs(_np(f.ctx).astype(np.float32) - _np(r.ctx).astype(np.float32)).max() <= ATTN_TOL
        for i in (0, 50, 127):
            assert torch.equal(f.k_cache[i].view(torch.int16), r.k_cache[i].view(torch.int16))
            assert torch.equal(f.v_cache[i].view(torch.int16), r.v_cache[i].view(torch.int16))


def test_decode_long_context_and_wide_batch(kv, ref):
    """Maximum sizes: one 40,000-key row (157 key ranges) next to short rows, and a 256-row batch."""
    case = DecodeCase([39999, 3, 20000, 511], seed=41)
    d = case.device()
    kv.append_decode(d.ctx, d.q, d.k, d.v, d.gate, d.q_norm_w, d.k_norm_w, d.cos, d.sin, d.pos_ids, d.seq_lens,
                     d.k_ptrs, d.v_ptrs, 0)
    torch.cuda.synchronize()
    assert torch.isfinite(d.ctx.float()).all()
    if ref is not None:
        r = case.device()
        ref.append(r.q, r.k, r.v, r.q_norm_w, r.k_norm_w, r.cos, r.sin, r.pos_ids, r.k_ptrs, r.v_ptrs, case.b)
        ref.decode_attention(r.ctx, r.q, r.gate, r.k_ptrs, r.v_ptrs, r.seq_lens, case.b, 0, 40000)
        torch.cuda.synchronize()
        assert np.abs(_np(d.ctx).astype(np.float32) - _np(r.ctx).astype(np.float32)).max() <= ATTN_TOL
    lens = np.random.default_rng(42).integers(1, 700, 256)
    case = DecodeCase(lens, seed=42)
    d = case.device()
    kv.append_decode(d.ctx, d.q, d.k, d.v, d.gate, d.q_norm_w, d.k_norm_w, d.cos, d.sin, d.pos_ids, d.seq_lens,
                     d.k_ptrs, d.v_ptrs, 256)
    torch.cuda.synchronize()
    if ref is not None:
        r = case.device()
        ref.append(r.q, r.k, r.v, r.q_norm_w, r.k_norm_w, r.cos, r.sin, r.pos_ids, r.k_ptrs, r.v_ptrs, 256)
        ref.decode_attention(r.ctx, r.q, r.gate, r.k_ptrs, r.v_ptrs, r.seq_lens, 256, 256, int(case.seq_lens.max()))
        torch.cuda.synchronize()
        assert np.abs(_np(d.ctx).astype(np.float32) - _np(r.ctx).astype(np.float32)).max() <= ATTN_TOL


def test_decode_maximum_batch_of_1024_rows(ref):
    """The largest batch one launch takes (1024 rows; the row tables live in shared memory): fused step against
    the reference's kernels, bytes of a row equal to the same row in a batch of 8, one row more is refused."""
    from oxide_infer_b200 import KvPath
    big = KvPath(0, max_batch=1024, max_seq_len=1024, max_prefill_rows=0)
    lens = np.random.default_rng(51).integers(1, 900, 1024)
    case = DecodeCase(lens, seed=51)
    d = case.device()
    big.append_decode(d.ctx, d.q, d.k, d.v, d.gate, d.q_norm_w, d.k_norm_w, d.cos, d.sin, d.pos_ids, d.seq_lens,
                      d.k_ptrs, d.v_ptrs, 0)
    torch.cuda.synchronize()
    assert big.device_status() == 0
    if ref is not None:
        r = case.device()
        ref.append(r.q, r.k, r.v, r.q_norm_w, r.k_norm_w, r.cos, r.sin, r.pos_ids, r.k_ptrs, r.v_ptrs, 1024)
        ref.decode_attention(r.ctx, r.q, r.gate, r.k_ptrs, r.v_ptrs, r.seq_lens, 1024, 0, int(case.seq_lens.max()))
        torch.cuda.synchronize()
        assert np.abs(_np(d.ctx).astype(np.float32) - _np(r.ctx).astype(np.float32)).max() <= ATTN_TOL
        for i in (0, 511, 1023):
            assert torch.equal(d.k_cache[i].view(torch.int16), r.k_cache[i].view(torch.int16))
    # rows 1000..1007 alone through the unfused pair: the same bytes as inside the batch of 1024
    a = case.device()
    big.append(a.q, a.k, a.v, a.q_norm_w, a.k_norm_w, a.cos, a.sin, a.pos_ids, a.k_ptrs, a.v_ptrs)
    sub = lambda t: t[1000:1008].contiguous()
    one = torch.zeros(8, NQ, HD, dtype=torch.float16, device="cuda")
    big.decode_attn(one, sub(a.q), sub(a.gate), sub(a.k_ptrs), sub(a.v_ptrs), sub(a.seq_lens), 0)
    torch.cuda.synchronize()
    assert torch.equal(one.view(torch.int16), d.ctx[1000:1008].view(torch.int16))
    with pytest.raises(Exception):
        KvPath(0, max_batch=1025, max_seq_len=64, max_prefill_rows=0)


@pytest.mark.parametrize("pinned", [True, False])
def test_host_buffer_step_equals_device_path(kv, pinned):
    """oxi_decode_step_host (q/k/v/gate, tables and positions in host memory, context back to the host, copies
    overlapped with the kernels on the library's own streams) gives the bytes of the per-layer device calls and
    leaves the same K/V rows - for three layers with their own caches and norm weights, twice in a row."""
    lens = [300, 1, 4095, 64, 777, 255]
    layers, b = 3, len(lens)
    cases = [DecodeCase(lens, seed=60 + l, max_pos=4100) for l in range(layers)]
    dev = [c.device() for c in cases]   # device path
    hst = [c.device() for c in cases]   # caches used by the host-buffer path
    for d in dev:
        kv.append_decode(d.ctx, d.q, d.k, d.v, d.gate, d.q_norm_w, d.k_norm_w, d.cos, d.sin, d.pos_ids, d.seq_lens,
                         d.k_ptrs, d.v_ptrs, 0)
    torch.cuda.synchronize()
    place = (lambda t: t.cpu().pin_memory()) if pinned else (lambda t: t.cpu())
    stack = lambda name: place(torch.stack([getattr(d, name) for d in hst]))
    hq, hk, hv, hg = stack("q"), stack("k"), stack("v"), stack("gate")
    hkp, hvp = stack("k_ptrs"), stack("v_ptrs")
    hpos = place(hst[0].pos_ids)
    qw = torch.stack([d.q_norm_w for d in hst]).contiguous()
    kw = torch.stack([d.k_norm_w for d in hst]).contiguous()
    hctx = torch.zeros(layers, b, NQ, HD, dtype=torch.float16)
    if pinned:
        hctx = hctx.pin_memory()
    for rep in range(2):  # the second call appends the same rows again: idempotent on the caches
        hctx.zero_()
        kv.decode_step_host(hctx, hq, hk, hv, hg, qw, kw, hst[0].cos, hst[0].sin, hpos, hkp, hvp, b, layers)
        torch.cuda.synchronize()
        for l in range(layers):
            assert torch.equal(hctx[l].view(torch.int16), dev[l].ctx.cpu().view(torch.int16))
            for i in (0, 2, 5):
                assert torch.equal(hst[l].k_cache[i].view(torch.int16), dev[l].k_cache[i].view(torch.int16))
                assert torch.equal(hst[l].v_cache[i].view(torch.int16), dev[l].v_cache[i].view(torch.int16))
    assert kv.device_status() == 0


def test_decode_step_replays_from_a_cuda_graph(kv):
    """The fused step (programmatic dependent launches included) can be captured once and replayed:
    a replay on fresh inputs equals the eager result byte for byte."""
    case = DecodeCase([300, 1200, 64, 2047], seed=43)
    e, g = case.device(), case.device()
    kv.append_decode(e.ctx, e.q, e.k, e.v, e.gate, e.q_norm_w, e.k_norm_w, e.cos, e.sin, e.pos_ids, e.seq_lens,
                     e.k_ptrs, e.v_ptrs, 0)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        # warm-up on the capture stream, then restore the cache rows the warm-up appended
        with torch.cuda.graph(graph, stream=side):
            kv.append_decode(g.ctx, g.q, g.k, g.v, g.gate, g.q_norm_w, g.k_norm_w, g.cos, g.sin, g.pos_ids,
                             g.seq_lens, g.k_ptrs, g.v_ptrs, 0)
    g.ctx.zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(e.ctx.view(torch.int16), g.ctx.view(torch.int16))
    for i in range(case.b):
        assert torch.equal(e.k_cache[i].view(torch.int16), g.k_cache[i].view(torch.int16))
    g.ctx.zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(e.ctx.view(torch.int16), g.ctx.view(torch.int16))


@pytest.mark.gpu
def test_graph_of_whole_step_replays_token_after_token_without_uploads():
    """A captured graph of (fused step of 3 layers + oxi_advance_step) replayed 12 times must leave
    the same caches and the same last ctx as 12 eager steps whose tables come from the host."""
    import torch
    from oxide_infer_b200 import KvPath
    steps, layers = 12, 3
    lens = [5, 250, 251, 1020]
    case = DecodeCase(lens, seed=71, spare_rows=steps + 1, max_pos=max(lens) + steps + 2)
    kv = KvPath(0, max_batch=8, max_seq_len=2048, max_prefill_rows=0)

    def fresh():
        ds = [case.device() for _ in range(layers)]
        return ds

    # eager: host-built tables per step
    de = fresh()
    for s in range(steps):
        pos = u32(case.lens + s)
        sl = u32(case.lens + s + 1)
        for l in range(layers):
            d = de[l]
            kv.append_decode(d.ctx, d.q, d.k, d.v, d.gate, d.q_norm_w, d.k_norm_w, d.cos, d.sin, pos, sl, d.k_ptrs, d.v_ptrs, 0)
    torch.cuda.synchronize()
    # graph: tables live on the device and advance there
    dg = fresh()
    pos, sl = u32(case.lens.copy()), u32(case.lens + 1)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        def step():
            for l in range(layers):
                d = dg[l]
                kv.append_decode(d.ctx, d.q, d.k, d.v, d.gate, d.q_norm_w, d.k_norm_w, d.cos, d.sin, pos, sl, d.k_ptrs, d.v_ptrs, 0)
            kv.advance_step(pos, sl, 1)
        step()  # the first token eagerly on the capture stream (also loads everything)
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            step()
        for _ in range(steps - 1):  # capturing records the step, it does not run it
            graph.replay()
    torch.cuda.synchronize()
    assert kv.device_status() == 0
    assert np.array_equal(pos.cpu().numpy().view(np.uint32), case.lens + steps)
    for l in range(layers):
        assert torch.equal(de[l].ctx.view(torch.int16), dg[l].ctx.view(torch.int16)), l
        for i in range(len(lens)):
            assert torch.equal(de[l].k_cache[i], dg[l].k_cache[i]), (l, i)
            assert torch.equal(de[l].v_cache[i], dg[l].v_cache[i]), (l, i)
