"""oxi_register_kv_slab: K/V rows inside the registered slab reach prefill attention through TMA tile
copies instead of per-thread copies.  Only the route into shared memory changes, so the context bytes
must be identical to those of a handle without a slab - for caches inside the slab, outside it, at an
offset that is not a whole number of rows, with ragged ends, windows, many runs per block and the
key-range split of small waves."""
import numpy as np
import pytest

from tests.kvcase import NKV, HD

pytestmark = pytest.mark.gpu

NQ = 16
ROW = NKV * HD  # f16 elements per cache row (1024 bytes)


def _wave(chunks, seed, outside=(), shifted=()):
    """chunks: (prefix, new rows) per request.  Caches are carved out of one slab, except the requests in
    `outside` (own allocation) and in `shifted` (inside the slab, 512 bytes off the row grid)."""
    import torch
    g = torch.Generator(device="cuda").manual_seed(seed)
    total = sum(p + n + 3 for p, n in chunks) * 2 + 8
    slab = torch.empty(total * ROW, dtype=torch.float16, device="cuda").normal_(generator=g)
    kc, vc, o = [], [], 2
    for i, (p, n) in enumerate(chunks):
        ln = p + n
        pair = []
        for _ in range(2):
            if i in outside:
                t = torch.empty(ln, NKV, HD, dtype=torch.float16, device="cuda").normal_(generator=g)
            else:
                start = o * ROW + (256 if i in shifted else 0)
                t = slab[start:start + ln * ROW].view(ln, NKV, HD)
                o += ln + 1 + (1 if i in shifted else 0)
            pair.append(t)
        kc.append(pair[0])
        vc.append(pair[1])
    rows = sum(n for _, n in chunks)
    q = torch.empty(rows, NQ, HD, dtype=torch.float16, device="cuda").normal_(generator=g)
    gate = torch.empty(rows, NQ, dtype=torch.float16, device="cuda").normal_(generator=g)
    owner = np.concatenate([np.full(n, i) for i, (_, n) in enumerate(chunks)])
    lens = np.concatenate([p + 1 + np.arange(n) for p, n in chunks]).astype(np.int32)
    kp = torch.tensor([kc[i].data_ptr() for i in owner], dtype=torch.int64, device="cuda")
    vp = torch.tensor([vc[i].data_ptr() for i in owner], dtype=torch.int64, device="cuda")
    return slab, q, gate, kp, vp, torch.from_numpy(lens).cuda(), rows, (kc, vc)  # the caches must stay alive


def _run(kv, w, window):
    import torch
    slab, q, gate, kp, vp, lens, rows, _keep = w
    ctx = torch.full((rows, NQ, HD), 3.0, dtype=torch.float16, device="cuda")
    kv.prefill_attn(ctx, q, gate, kp, vp, lens, window)
    torch.cuda.synchronize()
    return ctx


@pytest.fixture(scope="module")
def handles():
    from oxide_infer_b200 import KvPath
    return (KvPath(0, max_batch=8, max_seq_len=40960, max_prefill_rows=8192),
            KvPath(0, max_batch=8, max_seq_len=40960, max_prefill_rows=8192))


@pytest.mark.parametrize("window", [0, 300])
@pytest.mark.parametrize("chunks,outside,shifted", [
    ([(0, 64)], (), ()),                                        # one tile, ragged only
    ([(1000, 128)], (), ()),                                    # full tiles + ragged end
    ([(64, 64), (4000, 128), (129, 70), (2047, 1)], (), ()),    # several requests, a small wave (split)
    ([(500, 100), (700, 60), (300, 130)], (1,), (2,)),          # one cache outside the slab, one off the row grid
    ([(p, 128) for p in (8000, 100, 3000, 5555, 64, 7000, 1, 2500, 4096, 6000, 777, 1500,
                         3333, 8100, 900, 5000, 2000, 6500, 350, 7700)], (3,), (5,)),  # 40 blocks: no split
])
def test_tma_route_gives_identical_bytes(handles, chunks, outside, shifted, window):
    import torch
    tma, plain = handles
    w = _wave(chunks, seed=len(chunks) * 7 + window, outside=outside, shifted=shifted)
    tma.register_kv_slab(w[0])
    a = _run(tma, w, window)
    b = _run(plain, w, window)
    tma.register_kv_slab(None)
    c = _run(tma, w, window)
    assert tma.device_status() == 0 and plain.device_status() == 0
    assert torch.isfinite(a.float()).all()
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))
    assert torch.equal(c.view(torch.int16), b.view(torch.int16))


def test_slab_end_is_respected(handles):
    """A cache whose rows end exactly at the slab's last row, and one that runs past the registered bytes
    (the slab is registered shorter than the allocation): the second must take the per-thread path."""
    import torch
    tma, plain = handles
    w = _wave([(1000, 128), (2000, 64)], seed=3)
    slab = w[0]
    tma.register_kv_slab(slab[: (2 + 1128 + 1 + 1128 + 1 + 100) * ROW])  # ends inside the second request's K cache
    a = _run(tma, w, 0)
    tma.register_kv_slab(None)
    b = _run(plain, w, 0)
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))


def test_register_rejects_bad_arguments(handles):
    import torch
    tma, _ = handles
    t = torch.zeros(4096, dtype=torch.float16, device="cuda")
    with pytest.raises(Exception):
        tma.register_kv_slab(t[1:])      # 2 bytes off: not 16-byte aligned
    with pytest.raises(Exception):
        tma.register_kv_slab(t[:100])    # less than one row
    tma.register_kv_slab(None)
