"""The host side of the path through the C API (oxi_pool_*, oxi_tables_*): the slab pool with
its leases (kv_pool.rs:31-251) and the engine's per-step table build + upload
(batch_engine.rs:709-740), driven from ctypes the way a Rust FFI would.

Checks: the addressing formulas of kv_pool.rs:46-61; first-fit leases, coalescing release and
exhaustion; and three consecutive decode steps of a 4-layer model (conv, attention, conv,
attention) whose every pointer comes from the pool and the tables - upload for the first step,
oxi_tables_advance after it - byte-identical to the same steps with tables built in torch."""
import ctypes as C

import numpy as np
import pytest
import torch

from tests.kvcase import NQ, NKV, HD, HIDDEN, u32

pytestmark = pytest.mark.gpu


class Lease(C.Structure):
    _fields_ = [("tok_off", C.c_uint64), ("tokens", C.c_uint64), ("slot", C.c_uint64)]


class _Raw:
    """Device memory owned by the pool, seen as a torch tensor (CUDA array interface)."""

    def __init__(self, ptr, shape, typestr):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (int(ptr), False),
                                         "version": 2}


def view_f16(ptr, *shape):
    return torch.as_tensor(_Raw(ptr, shape, "<f2"), device="cuda")


def view_at(ptr, nbytes, dtype, count):
    return torch.as_tensor(_Raw(ptr, (count,), {torch.int64: "<i8", torch.int32: "<i4"}[dtype]), device="cuda")


@pytest.fixture(scope="module")
def lib():
    from oxide_infer_b200 import _lib, build
    build.build()
    return _lib.load()


IS_CONV = [1, 0, 1, 0]  # two conv and two attention layers
CAP = 16384


def _pool(lib, max_batch=8, cap=CAP):
    p = C.c_void_p()
    kinds = (C.c_uint8 * len(IS_CONV))(*IS_CONV)
    assert lib.oxi_pool_create(C.byref(p), kinds, len(IS_CONV), max_batch, cap) == 0, lib.oxi_host_last_error_string()
    return p


def test_pool_leases_addressing_and_exhaustion(lib):
    torch.zeros(1, device="cuda")
    pool = _pool(lib, max_batch=3)
    st = torch.cuda.current_stream().cuda_stream
    assert lib.oxi_pool_capacity_tokens(pool) == CAP and lib.oxi_pool_free_tokens(pool) == CAP
    a, b, c, d = Lease(), Lease(), Lease(), Lease()
    assert lib.oxi_pool_acquire(pool, st, 1000, C.byref(a)) == 0
    assert lib.oxi_pool_acquire(pool, st, 5000, C.byref(b)) == 0
    assert (a.tok_off, a.tokens, b.tok_off) == (0, 1000, 1000) and a.slot != b.slot   # first fit, distinct slots
    # kv_pool.rs:46-61: plane 2a is K of attention layer a, plane 2a+1 its V; rows of 1024 bytes
    k1a, v1a = lib.oxi_pool_k_ptr(pool, 1, C.byref(a)), lib.oxi_pool_v_ptr(pool, 1, C.byref(a))
    k3a, k1b = lib.oxi_pool_k_ptr(pool, 3, C.byref(a)), lib.oxi_pool_k_ptr(pool, 1, C.byref(b))
    assert v1a - k1a == CAP * 1024 and k3a - k1a == 2 * CAP * 1024 and k1b - k1a == 1000 * 1024
    assert lib.oxi_pool_k_ptr(pool, 0, C.byref(a)) == 0 and lib.oxi_pool_conv_ptr(pool, 1, C.byref(a)) == 0  # wrong kind
    c0a, c2a = lib.oxi_pool_conv_ptr(pool, 0, C.byref(a)), lib.oxi_pool_conv_ptr(pool, 2, C.byref(a))
    c0b = lib.oxi_pool_conv_ptr(pool, 0, C.byref(b))
    plane = HIDDEN * 6 * 2
    assert c2a - c0a == plane and abs(c0b - c0a) == 2 * plane * abs(int(b.slot) - int(a.slot))
    # the slot's conv states are zeroed by acquire
    torch.cuda.synchronize()
    assert view_f16(c0a, HIDDEN, 6).abs().sum().item() == 0
    # exhaustion: rows (first), then slots
    assert lib.oxi_pool_acquire(pool, st, CAP, C.byref(c)) == -4 and b"free" in lib.oxi_host_last_error_string()
    assert lib.oxi_pool_acquire(pool, st, 100, C.byref(c)) == 0
    assert lib.oxi_pool_acquire(pool, st, 100, C.byref(d)) == -4                       # no conv slot left
    assert lib.oxi_pool_free_slots(pool) == 0
    # release coalesces: freeing a and b (neighbours) leaves one hole of 6000 rows that a 6000-row lease fits
    assert lib.oxi_pool_release(pool, C.byref(a)) == 0 and lib.oxi_pool_release(pool, C.byref(b)) == 0
    assert lib.oxi_pool_free_tokens(pool) == CAP - 100
    assert lib.oxi_pool_acquire(pool, st, 6000, C.byref(d)) == 0 and d.tok_off == 0
    bad = Lease(CAP, 10, 0)
    assert lib.oxi_pool_release(pool, C.byref(bad)) == -3
    assert lib.oxi_pool_destroy(pool) == 0


def test_decode_steps_through_pool_and_tables_equal_direct_calls(lib):
    from oxide_infer_b200 import KvPath
    from oracle import cpu as O
    rng = np.random.default_rng(17)
    lens = [300, 5, 1023, 64, 700]
    steps, b = 3, len(lens)
    kv = KvPath(0, max_batch=8, max_seq_len=2048, max_prefill_rows=0)
    pool = _pool(lib)
    st = torch.cuda.current_stream().cuda_stream
    leases = []
    for n in lens:
        l = Lease()
        assert lib.oxi_pool_acquire(pool, st, n + steps, C.byref(l)) == 0
        leases.append(l)
    f16 = lambda *s, sc=1.0: torch.from_numpy((rng.standard_normal(s, dtype=np.float32) * sc).astype(np.float16)).cuda()
    # fill the leased K/V rows and conv states; keep copies for the direct path
    direct = {}
    for layer, conv in enumerate(IS_CONV):
        for i, (n, l) in enumerate(zip(lens, leases)):
            if conv:
                s = f16(HIDDEN, 6)
                view_f16(lib.oxi_pool_conv_ptr(pool, layer, C.byref(l)), HIDDEN, 6).copy_(s)
                direct[(layer, i)] = s.clone()
            else:
                k, v = f16(n + steps, NKV, HD), f16(n + steps, NKV, HD)
                view_f16(lib.oxi_pool_k_ptr(pool, layer, C.byref(l)), n + steps, NKV, HD).copy_(k)
                view_f16(lib.oxi_pool_v_ptr(pool, layer, C.byref(l)), n + steps, NKV, HD).copy_(v)
                direct[(layer, i)] = (k.clone(), v.clone())
    q, k_in, v_in, gate = f16(b, NQ, HD), f16(b, NKV, HD), f16(b, NKV, HD), f16(b, NQ)
    bcx, conv_w = f16(b, 3 * HIDDEN), f16(HIDDEN, 7, sc=0.1)
    qw = torch.from_numpy((1 + 0.02 * rng.standard_normal(HD)).astype(np.float16)).cuda()
    kw = torch.from_numpy((1 + 0.02 * rng.standard_normal(HD)).astype(np.float16)).cuda()
    cos, sin = (torch.from_numpy(t).cuda() for t in O.rope_table(max(lens) + steps + 2, 1e6, 0.5))

    tables = C.c_void_p()
    assert lib.oxi_tables_create(C.byref(tables), pool, 8) == 0
    for i, (n, l) in enumerate(zip(lens, leases)):
        assert lib.oxi_tables_set_row(tables, i, C.byref(l), n) == 0
    assert lib.oxi_tables_set_row(tables, 0, C.byref(leases[1]), lens[1] + steps) == -3   # position beyond the lease
    assert lib.oxi_tables_set_row(tables, 0, C.byref(leases[0]), lens[0]) == 0
    assert lib.oxi_tables_upload(tables, st, b) == 0 and lib.oxi_tables_batch(tables) == b
    out_t = []
    for s in range(steps):
        for layer, conv in enumerate(IS_CONV):
            if conv:
                y = torch.zeros(b, HIDDEN, dtype=torch.float16, device="cuda")
                assert lib.oxi_conv_decode(kv.h, st, y.data_ptr(), lib.oxi_tables_conv_ptrs(tables, layer), bcx.data_ptr(),
                                           conv_w.data_ptr(), b) == 0
                out_t.append(y)
            else:
                ctx = torch.zeros(b, NQ, HD, dtype=torch.float16, device="cuda")
                assert lib.oxi_append_decode(kv.h, st, ctx.data_ptr(), q.data_ptr(), k_in.data_ptr(), v_in.data_ptr(),
                                             gate.data_ptr(), qw.data_ptr(), kw.data_ptr(), cos.data_ptr(), sin.data_ptr(),
                                             lib.oxi_tables_pos_ids(tables), lib.oxi_tables_seq_lens(tables),
                                             lib.oxi_tables_k_ptrs(tables, layer), lib.oxi_tables_v_ptrs(tables, layer),
                                             b, 0, 1e-5) == 0
                out_t.append(ctx)
        assert lib.oxi_tables_advance(kv.h, tables, st, 1) == 0   # no upload for the next step
    torch.cuda.synchronize()

    # the same steps with tables built in torch over the copies
    out_d = []
    for s in range(steps):
        pos, sl = u32(np.asarray(lens, np.uint32) + s), u32(np.asarray(lens, np.uint32) + s + 1)
        for layer, conv in enumerate(IS_CONV):
            if conv:
                y = torch.zeros(b, HIDDEN, dtype=torch.float16, device="cuda")
                ptrs = torch.tensor([direct[(layer, i)].data_ptr() for i in range(b)], dtype=torch.int64, device="cuda")
                kv.conv_decode(y, ptrs, bcx, conv_w)
                out_d.append(y)
            else:
                ctx = torch.zeros(b, NQ, HD, dtype=torch.float16, device="cuda")
                kp = torch.tensor([direct[(layer, i)][0].data_ptr() for i in range(b)], dtype=torch.int64, device="cuda")
                vp = torch.tensor([direct[(layer, i)][1].data_ptr() for i in range(b)], dtype=torch.int64, device="cuda")
                kv.append_decode(ctx, q, k_in, v_in, gate, qw, kw, cos, sin, pos, sl, kp, vp, 0)
                out_d.append(ctx)
    torch.cuda.synchronize()
    assert kv.device_status() == 0
    for i, (x, y) in enumerate(zip(out_t, out_d)):
        assert torch.equal(x.view(torch.int16), y.view(torch.int16)), i
    for layer, conv in enumerate(IS_CONV):
        for i, (n, l) in enumerate(zip(lens, leases)):
            if conv:
                got = view_f16(lib.oxi_pool_conv_ptr(pool, layer, C.byref(l)), HIDDEN, 6)
                assert torch.equal(got.view(torch.int16), direct[(layer, i)].view(torch.int16))
            else:
                got = view_f16(lib.oxi_pool_k_ptr(pool, layer, C.byref(l)), n + steps, NKV, HD)
                assert torch.equal(got.view(torch.int16), direct[(layer, i)][0].view(torch.int16))
    # a second upload right behind the first (no sync) and the positions the host image followed
    for i, (n, l) in enumerate(zip(lens, leases)):
        assert lib.oxi_tables_set_row(tables, i, C.byref(l), n + 1) == 0
    for _ in range(6):
        assert lib.oxi_tables_upload(tables, st, b) == 0
    torch.cuda.synchronize()
    pos_now = view_at(lib.oxi_tables_pos_ids(tables), 4 * b, torch.int32, b).cpu().numpy()
    assert np.array_equal(pos_now, np.asarray(lens) + 1)
    assert lib.oxi_tables_destroy(tables) == 0
    for l in leases:
        assert lib.oxi_pool_release(pool, C.byref(l)) == 0
    assert lib.oxi_pool_free_tokens(pool) == lib.oxi_pool_capacity_tokens(pool)
    assert lib.oxi_pool_destroy(pool) == 0
    kv.close()
