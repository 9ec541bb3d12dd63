"""oxi_project_append: the q/k/v/gate projection GEMMs (batch_engine.rs:914-926) with the append operator
(batch_engine.rs:941-1014) as the GEMM's epilogue, and oxi_linear_forward (o_proj, batch_engine.rs:1241-1245).

Bars:
  * the f16 projections are within one f16 step of an fp32-accumulated matmul (torch float32 on the GPU and
    the CPU oracle's orc_linear_f16), nearly all of them bit-identical;
  * given those projections, q and the K/V cache rows are the BYTES oxi_append writes, and through it the
    bytes of the reference's own six kernels;
  * decode attention after the fused kernel equals the fused append+attention step on the same projections."""
import numpy as np
import pytest
import torch

from tests.kvcase import NQ, NKV, HD, HIDDEN, DecodeCase, guarded, ulp_diff_f16

pytestmark = pytest.mark.gpu

NOUT = NQ * HD + 2 * NKV * HD + NQ


def _assert_same_projections(got, want):
    """Two f32-accumulated GEMMs differ by their summation order only: a few 1e-6 absolute on sums of 2048
    products of size ~1e-2.  After rounding to f16 that is at most one f16 step, except for values near zero,
    whose f16 steps are finer than the accumulation noise: there the absolute difference is bounded instead."""
    g, w = got.astype(np.float32), want.astype(np.float32)
    ulp = ulp_diff_f16(got, want)
    ok = (ulp <= 1) | (np.abs(g - w) <= 3e-5)
    assert ok.all(), (int(ulp.max()), float(np.abs(g - w).max()))
    assert (ulp != 0).mean() < 0.03, float((ulp != 0).mean())  # measured: about 1 % land on the other side of a rounding boundary
    return ulp


@pytest.fixture(scope="module")
def kv():
    from oxide_infer_b200 import KvPath, build
    build.build()
    p = KvPath(0, max_batch=1024, max_seq_len=8192, max_prefill_rows=4096)
    yield p
    assert p.device_status() == 0
    p.close()


def _weights(seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    rn = lambda o: (torch.randn(o, HIDDEN, device="cuda", generator=g) * HIDDEN ** -0.5).half()
    return rn(NQ * HD), rn(NKV * HD), rn(NKV * HD), rn(NQ)


def _project(kv, case, x, ws, raw=True):
    from oxide_infer_b200 import Linear
    lin = Linear(*ws)
    d = case.device()
    rows = x.shape[0]
    q_out = guarded(np.zeros((rows, NQ, HD), np.float16), "q_out")
    gate_out = guarded(np.zeros((rows, NQ), np.float16), "gate_out")
    raw_out = guarded(np.zeros((rows, NOUT), np.float16), "raw_out") if raw else None
    kv.project_append(lin, x, q_out, gate_out, d.q_norm_w, d.k_norm_w, d.cos, d.sin, d.pos_ids, d.k_ptrs, d.v_ptrs,
                      raw_out=raw_out)
    torch.cuda.synchronize()
    return d, q_out, gate_out, raw_out


# up to 512 rows run the four-CTA cluster kernel (one to four row tiles), more rows the persistent 128 x 256 kernel
@pytest.mark.parametrize("lens", [[5], [300, 1, 64, 777, 31, 2047, 512], list(range(100, 228)), list(range(10, 266)),
                                  list(range(10, 267)), list(range(10, 310)), list(range(10, 522)), list(range(10, 523)),
                                  list(range(10, 650))])
def test_project_append_equals_matmul_then_append(kv, ref, lens):
    b = len(lens)
    case = DecodeCase(lens, seed=80 + b)
    g = torch.Generator(device="cuda").manual_seed(b)
    x = torch.randn(b, HIDDEN, device="cuda", generator=g).half()
    ws = _weights(1000 + b)
    d, q_out, gate_out, raw = _project(kv, case, x, ws)
    # (1) projections vs an fp32-accumulated matmul
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    want = torch.cat([(x.float() @ w.float().t()) for w in ws], dim=1).half()
    torch.backends.cuda.matmul.allow_tf32 = prev
    _assert_same_projections(raw.cpu().numpy(), want.cpu().numpy())
    assert torch.equal(gate_out.view(torch.int16), raw[:, 3072:].contiguous().view(torch.int16))
    # (2) the same f16 projections through oxi_append: q and the cache rows must be the same bytes
    a = case.device()
    q = raw[:, :2048].contiguous().view(b, NQ, HD).clone()
    k = raw[:, 2048:2560].contiguous().view(b, NKV, HD)
    v = raw[:, 2560:3072].contiguous().view(b, NKV, HD)
    kv.append(q, k, v, a.q_norm_w, a.k_norm_w, a.cos, a.sin, a.pos_ids, a.k_ptrs, a.v_ptrs)
    torch.cuda.synchronize()
    assert torch.equal(q.view(torch.int16), q_out.view(torch.int16))
    for i in range(b):
        assert torch.equal(a.k_cache[i].view(torch.int16), d.k_cache[i].view(torch.int16)), i
        assert torch.equal(a.v_cache[i].view(torch.int16), d.v_cache[i].view(torch.int16)), i
    # (3) and through the reference's six kernels
    if ref is not None and b <= 128:
        r = case.device()
        rq = raw[:, :2048].contiguous().view(b, NQ, HD).clone()
        rk = k.clone()
        ref.append(rq, rk, v, r.q_norm_w, r.k_norm_w, r.cos, r.sin, r.pos_ids, r.k_ptrs, r.v_ptrs, b)
        torch.cuda.synchronize()
        assert torch.equal(rq.view(torch.int16), q_out.view(torch.int16))
        for i in (0, b // 2, b - 1):
            assert torch.equal(r.k_cache[i].view(torch.int16), d.k_cache[i].view(torch.int16))
    # (4) attention after the fused kernel = the fused append + attention step on the same projections
    ctx = torch.zeros(b, NQ, HD, dtype=torch.float16, device="cuda")
    kv.decode_attn(ctx, q_out, gate_out, d.k_ptrs, d.v_ptrs, d.seq_lens, 0)
    f = case.device()
    qr = raw[:, :2048].contiguous().view(b, NQ, HD)
    kv.append_decode(f.ctx, qr, k, v, gate_out, f.q_norm_w, f.k_norm_w, f.cos, f.sin, f.pos_ids, f.seq_lens,
                     f.k_ptrs, f.v_ptrs, 0)
    torch.cuda.synchronize()
    assert torch.equal(ctx.view(torch.int16), f.ctx.view(torch.int16))


def test_projections_against_the_cpu_oracle(kv):
    from oracle import cpu as O
    O.build()
    O.use_all_cores()
    lens = [40, 3, 500, 129, 64, 1000]
    case = DecodeCase(lens, seed=7)
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(len(lens), HIDDEN, device="cuda", generator=g).half()
    ws = _weights(3)
    d, q_out, gate_out, raw = _project(kv, case, x, ws)
    xn = x.cpu().numpy()
    want = np.concatenate([O.linear(xn, w.cpu().numpy()) for w in ws], axis=1)
    ulp = _assert_same_projections(raw.cpu().numpy(), want)
    # the oracle's append on ITS projections: K within one f16 step (a last-bit difference of a projection moves
    # the normalised value by at most that), V bit-exact wherever the projections agree
    h = case.host()
    q = want[:, :2048].reshape(-1, NQ, HD).copy()
    k = want[:, 2048:2560].reshape(-1, NKV, HD).copy()
    v = want[:, 2560:3072].reshape(-1, NKV, HD).copy()
    O.qk_rmsnorm(q, case.q_norm_w)
    O.qk_rmsnorm(k, case.k_norm_w)
    O.rope(q, case.cos, case.sin, case.pos_ids)
    O.rope(k, case.cos, case.sin, case.pos_ids)
    assert np.abs(q_out.cpu().numpy().astype(np.float32) - q.astype(np.float32)).max() <= 4e-3
    for i, n in enumerate(lens):
        got = d.k_cache[i][n].cpu().numpy().astype(np.float32)
        assert np.abs(got - k[i].astype(np.float32)).max() <= 4e-3
        same = ulp[i, 2560:3072] == 0
        assert np.array_equal(d.v_cache[i][n].cpu().numpy().reshape(-1)[same], v[i].reshape(-1)[same])


def test_prefill_wave_shape_and_untouched_rows(kv):
    """4,096 wave rows (32 requests x 128 tokens): every row lands at its own position of its request's cache and
    nothing else in the caches changes."""
    from oxide_infer_b200 import Linear
    nseq, new = 32, 128
    rows = nseq * new
    rng = np.random.default_rng(9)
    prefix = rng.integers(0, 300, nseq)
    g = torch.Generator(device="cuda").manual_seed(9)
    kc = [guarded(np.full((int(p) + new, NKV, HD), 7.0, np.float16), f"k{i}") for i, p in enumerate(prefix)]
    vc = [guarded(np.full((int(p) + new, NKV, HD), 7.0, np.float16), f"v{i}") for i, p in enumerate(prefix)]
    owner = np.repeat(np.arange(nseq), new)
    pos = (prefix[owner] + np.tile(np.arange(new), nseq)).astype(np.int32)
    kp = torch.tensor([kc[i].data_ptr() for i in owner], dtype=torch.int64, device="cuda")
    vp = torch.tensor([vc[i].data_ptr() for i in owner], dtype=torch.int64, device="cuda")
    dpos = torch.from_numpy(pos).cuda()
    x = torch.randn(rows, HIDDEN, device="cuda", generator=g).half()
    ws = _weights(11)
    lin = Linear(*ws)
    case = DecodeCase([1], seed=1, max_pos=512)
    c = case.device()
    q_out = torch.zeros(rows, NQ, HD, dtype=torch.float16, device="cuda")
    gate_out = torch.zeros(rows, NQ, dtype=torch.float16, device="cuda")
    raw = torch.zeros(rows, NOUT, dtype=torch.float16, device="cuda")
    kv.project_append(lin, x, q_out, gate_out, c.q_norm_w, c.k_norm_w, c.cos, c.sin, dpos, kp, vp, raw_out=raw)
    q = raw[:, :2048].contiguous().view(rows, NQ, HD).clone()
    k = raw[:, 2048:2560].contiguous().view(rows, NKV, HD)
    v = raw[:, 2560:3072].contiguous().view(rows, NKV, HD)
    ka = [torch.full_like(t, 7.0) for t in kc]
    va = [torch.full_like(t, 7.0) for t in vc]
    kpa = torch.tensor([ka[i].data_ptr() for i in owner], dtype=torch.int64, device="cuda")
    vpa = torch.tensor([va[i].data_ptr() for i in owner], dtype=torch.int64, device="cuda")
    kv.append(q, k, v, c.q_norm_w, c.k_norm_w, c.cos, c.sin, dpos, kpa, vpa, batch=rows)
    torch.cuda.synchronize()
    assert torch.equal(q.view(torch.int16), q_out.view(torch.int16))
    for i in range(nseq):
        assert torch.equal(ka[i].view(torch.int16), kc[i].view(torch.int16)), i   # new rows equal, prefix rows still 7.0
        assert torch.equal(va[i].view(torch.int16), vc[i].view(torch.int16)), i


@pytest.mark.parametrize("rows,out", [(1, 2048), (128, 2048), (300, 2048), (7, 16), (130, 520), (300, 520), (513, 16),
                                      (1000, 3088)])
def test_linear_forward(kv, rows, out):
    from oxide_infer_b200 import Linear
    g = torch.Generator(device="cuda").manual_seed(rows + out)
    w = (torch.randn(out, HIDDEN, device="cuda", generator=g) * HIDDEN ** -0.5).half()
    x = torch.randn(rows, HIDDEN, device="cuda", generator=g).half()
    y = guarded(np.zeros((rows, out), np.float16), "y")
    kv.linear(Linear(w), x, y)
    torch.cuda.synchronize()
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    want = (x.float() @ w.float().t()).half()
    torch.backends.cuda.matmul.allow_tf32 = prev
    _assert_same_projections(y.cpu().numpy(), want.cpu().numpy())


def test_argument_errors(kv):
    from oxide_infer_b200 import Linear, OxiError
    ws = _weights(1)
    lin, plain = Linear(*ws), Linear(ws[0])
    case = DecodeCase([3, 4], seed=2)
    d = case.device()
    x = torch.zeros(2, HIDDEN, dtype=torch.float16, device="cuda")
    q_out, gate_out = torch.zeros(2, NQ, HD, dtype=torch.float16, device="cuda"), torch.zeros(2, NQ, dtype=torch.float16, device="cuda")
    with pytest.raises(OxiError):   # a plain matrix where the four projections are expected
        kv.project_append(plain, x, q_out, gate_out, d.q_norm_w, d.k_norm_w, d.cos, d.sin, d.pos_ids, d.k_ptrs, d.v_ptrs)
    with pytest.raises(OxiError):
        kv.linear(lin, x, torch.zeros(2, 2048, dtype=torch.float16, device="cuda"))
    with pytest.raises(OxiError):   # more rows than the handle was created for
        kv.project_append(lin, x, q_out, gate_out, d.q_norm_w, d.k_norm_w, d.cos, d.sin, d.pos_ids, d.k_ptrs, d.v_ptrs,
                          rows=5000)
    # a misaligned cache pointer is reported and that row's K/V are not written
    bad = d.k_ptrs.clone()
    bad[1] += 2
    kv.project_append(lin, x, q_out, gate_out, d.q_norm_w, d.k_norm_w, d.cos, d.sin, d.pos_ids, bad, d.v_ptrs)
    torch.cuda.synchronize()
    assert kv.device_status() == 1
    assert torch.equal(d.k_cache[1].cpu(), torch.from_numpy(case.k_cache[1]))


def test_wave_kernel_skips_rows_with_misaligned_cache_pointers(kv):
    """More than 512 rows run the CTA-pair kernel: a K pointer and a V pointer that are not 16-byte aligned are reported, those
    two cache rows stay untouched, every other row is written as by the aligned call."""
    from oxide_infer_b200 import Linear
    lens = list(range(20, 620))
    case = DecodeCase(lens, seed=91)
    b = len(lens)
    g = torch.Generator(device="cuda").manual_seed(91)
    x = torch.randn(b, HIDDEN, device="cuda", generator=g).half()
    lin = Linear(*_weights(91))
    good, d = case.device(), case.device()
    outs = [torch.zeros(b, NQ, HD, dtype=torch.float16, device="cuda") for _ in range(2)]
    gates = [torch.zeros(b, NQ, dtype=torch.float16, device="cuda") for _ in range(2)]
    kv.project_append(lin, x, outs[0], gates[0], good.q_norm_w, good.k_norm_w, good.cos, good.sin, good.pos_ids, good.k_ptrs, good.v_ptrs)
    torch.cuda.synchronize()
    assert kv.device_status() == 0
    bad_k, bad_v = d.k_ptrs.clone(), d.v_ptrs.clone()
    bad_k[300] += 2
    bad_v[599] += 6
    kv.project_append(lin, x, outs[1], gates[1], d.q_norm_w, d.k_norm_w, d.cos, d.sin, d.pos_ids, bad_k, bad_v)
    torch.cuda.synchronize()
    assert kv.device_status() == 1
    assert torch.equal(outs[0].view(torch.int16), outs[1].view(torch.int16))
    assert torch.equal(gates[0].view(torch.int16), gates[1].view(torch.int16))
    for i in range(b):
        want_k = torch.from_numpy(case.k_cache[i]).cuda() if i == 300 else good.k_cache[i]
        want_v = torch.from_numpy(case.v_cache[i]).cuda() if i == 599 else good.v_cache[i]
        assert torch.equal(d.k_cache[i].view(torch.int16), want_k.view(torch.int16)), i
        assert torch.equal(d.v_cache[i].view(torch.int16), want_v.view(torch.int16)), i
