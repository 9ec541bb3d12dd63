"""Key-range split of small prefill waves (oxi_prefill_split_configure): a wave with fewer
(64-row block, KV head) items than SMs cuts its long blocks into parts and merges the parts'
partial softmax results.  The split changes only the order of the sums: results must stay within
the attention tolerance of the oracle and very close to the unsplit kernel; waves that do not
qualify (too large, not enough reserved slots, split turned off) must be bit-identical to the
unsplit kernel; the paged layout must give the same bits as the pointer tables."""
import numpy as np
import pytest

from oracle import cpu as O
from tests.kvcase import NKV, HD

pytestmark = pytest.mark.gpu

NQ = 16
ATTN_TOL = 2e-3  # max abs error of the attention output against the reference algorithm


class Wave:
    """chunks: (prefix, new rows) per request; every request has its own contiguous cache."""

    def __init__(self, chunks, seed, kscale=1.0):
        import torch
        self.chunks = chunks
        self.rows = sum(n for _, n in chunks)
        g = torch.Generator(device="cuda").manual_seed(seed)
        rn = lambda *s, sc=1.0: (torch.empty(*s, dtype=torch.float32, device="cuda").normal_(generator=g) * sc).half()
        self.kc = [rn(p + n, NKV, HD, sc=kscale) for p, n in chunks]
        self.vc = [rn(p + n, NKV, HD) for p, n in chunks]
        self.q, self.gate = rn(self.rows, NQ, HD), rn(self.rows, NQ)
        self.owner = np.concatenate([np.full(n, i) for i, (_, n) in enumerate(chunks)])
        self.lens = np.concatenate([p + 1 + np.arange(n) for p, n in chunks]).astype(np.int32)
        self.kp = torch.tensor([self.kc[i].data_ptr() for i in self.owner], dtype=torch.int64, device="cuda")
        self.vp = torch.tensor([self.vc[i].data_ptr() for i in self.owner], dtype=torch.int64, device="cuda")
        self.dlen = torch.from_numpy(self.lens).cuda()

    def run(self, kv, window, lens=None):
        import torch
        ctx = torch.full((self.rows, NQ, HD), 7.0, dtype=torch.float16, device="cuda")
        kv.prefill_attn(ctx, self.q, self.gate, self.kp, self.vp, self.dlen if lens is None else lens, window)
        torch.cuda.synchronize()
        return ctx

    def oracle(self, window, lens=None):
        ks = [k.cpu().numpy() for k in self.kc]
        vs = [v.cpu().numpy() for v in self.vc]
        hk, hv = O.ptr_table([ks[i] for i in self.owner]), O.ptr_table([vs[i] for i in self.owner])
        want = O.attn_online(self.q.cpu().numpy(), hk, hv, (self.lens if lens is None else lens).astype(np.uint32), window)
        O.sigmoid_gate(want, self.gate.cpu().numpy())
        return want.astype(np.float32)


@pytest.fixture(scope="module")
def kvs():
    """(split handle, plain handle)"""
    from oxide_infer_b200 import KvPath
    a = KvPath(0, max_batch=8, max_seq_len=40960, max_prefill_rows=4096)
    a.prefill_split_configure(256, 256)
    b = KvPath(0, max_batch=8, max_seq_len=40960, max_prefill_rows=4096)
    b.prefill_split_configure(0, 0)  # the split is on by default
    return a, b


@pytest.mark.parametrize("window", [0, 256, 1000])
@pytest.mark.parametrize("chunks", [[(4000, 128)], [(0, 5), (77, 1), (3, 30), (1000, 64)], [(2049, 129), (333, 70)],
                                    [(20000, 17)]])
def test_split_wave_matches_oracle_and_unsplit(kvs, chunks, window):
    split, plain = kvs
    w = Wave(chunks, seed=len(chunks) + window)
    a, b = w.run(split, window), w.run(plain, window)
    assert split.device_status() == 0
    want = w.oracle(window)
    fa, fb = a.float().cpu().numpy(), b.float().cpu().numpy()
    assert np.abs(fa - want).max() <= ATTN_TOL
    assert np.abs(fa - fb).max() <= 1e-3  # same products, another order of the f32 sums


def test_split_really_splits(kvs):
    """A block far longer than part_keys: the merged result differs from the unsplit bits somewhere
    (another summation order), which shows the split path ran, and stays within the tolerance."""
    import torch
    split, plain = kvs
    w = Wave([(30000, 64)], seed=5)
    a, b = w.run(split, 0), w.run(plain, 0)
    assert np.abs(a.float().cpu().numpy() - b.float().cpu().numpy()).max() <= 1e-3
    assert not torch.equal(a.view(torch.int16), b.view(torch.int16))


def test_large_scores_keep_the_reference_maximum_consistent(kvs):
    """Keys scaled so that row maxima differ a lot between parts: the merge weights 2^(m_s - m) matter."""
    split, plain = kvs
    w = Wave([(6000, 64)], seed=9, kscale=4.0)
    a = w.run(split, 0).float().cpu().numpy()
    assert np.abs(a - w.oracle(0)).max() <= ATTN_TOL


def test_skipped_rows_stay_untouched(kvs):
    """seq_len 0 rows are skipped (status bit) and their output is not written, also by the merge."""
    import torch
    split, _ = kvs
    w = Wave([(5000, 64)], seed=11)
    lens = w.lens.copy()
    lens[[3, 40]] = 0
    a = w.run(split, 0, lens=torch.from_numpy(lens).cuda())
    assert split.device_status() & 2  # OXI_DEV_BAD_SEQ_LEN (reading clears it)
    assert bool((a[[3, 40]] == 7.0).all())
    keep = np.setdiff1d(np.arange(64), [3, 40])
    want = w.oracle(0, lens=np.where(lens == 0, 1, lens))
    assert np.abs(a.float().cpu().numpy()[keep] - want[keep]).max() <= ATTN_TOL


def test_waves_that_do_not_qualify_are_bit_identical(kvs):
    import torch
    from oxide_infer_b200 import KvPath
    split, plain = kvs
    # 40 blocks x 4 KV heads >= SMs: runs unsplit
    w = Wave([(3000, 128)] * 20, seed=13)
    assert torch.equal(w.run(split, 0).view(torch.int16), w.run(plain, 0).view(torch.int16))
    # more parts than reserved slots: runs unsplit
    few = KvPath(0, max_batch=8, max_seq_len=40960, max_prefill_rows=4096)
    # a new handle splits by default, with a reservation no split wave can exceed
    w = Wave([(4000, 128)], seed=14)
    assert not torch.equal(w.run(few, 0).view(torch.int16), w.run(plain, 0).view(torch.int16))
    assert np.abs(w.run(few, 0).float().cpu().numpy() - w.oracle(0)).max() <= ATTN_TOL
    few.prefill_split_configure(256, 4)
    w = Wave([(4000, 128)], seed=14)
    assert torch.equal(w.run(few, 0).view(torch.int16), w.run(plain, 0).view(torch.int16))
    # enough now; then off again
    few.prefill_split_configure(256, 64)
    assert not torch.equal(w.run(few, 0).view(torch.int16), w.run(plain, 0).view(torch.int16))
    before = few.workspace_bytes
    few.prefill_split_configure(0, 0)
    assert few.workspace_bytes == before - 64 * few.prefill_split_slot_bytes() - 3 * 1024 * 32 * 4
    assert torch.equal(w.run(few, 0).view(torch.int16), w.run(plain, 0).view(torch.int16))


def test_configure_rejects_bad_arguments(kvs):
    split, _ = kvs
    with pytest.raises(Exception):
        split.prefill_split_configure(100, 16)
    with pytest.raises(Exception):
        split.prefill_split_configure(256, 100000)


@pytest.mark.parametrize("block_size,window", [(16, 0), (128, 300)])
def test_paged_split_equals_pointer_table_split(kvs, block_size, window):
    import torch
    from oxide_infer_b200 import PagedLayout
    split, _ = kvs
    rng = np.random.default_rng(21)
    chunks = [(5000, 64), (1234, 100)]
    w = Wave(chunks, seed=21)
    a = w.run(split, window)
    need = [(p + n + block_size - 1) // block_size for p, n in chunks]
    total = sum(need) + 2
    perm = rng.permutation(total).astype(np.int32)
    tables = np.zeros((len(chunks), max(need)), np.int32)
    kpool = torch.zeros(total, block_size, NKV, HD, dtype=torch.float16, device="cuda")
    vpool = torch.zeros_like(kpool)
    o = 0
    for i, (p, n) in enumerate(chunks):
        ids = perm[o:o + need[i]]
        o += need[i]
        tables[i, :need[i]] = ids
        for j, bid in enumerate(ids):
            lo, hi = j * block_size, min((j + 1) * block_size, p + n)
            kpool[bid, :hi - lo] = w.kc[i][lo:hi]
            vpool[bid, :hi - lo] = w.vc[i][lo:hi]
    lay = PagedLayout.of(kpool, vpool, torch.from_numpy(tables).cuda(), block_size)
    b = torch.zeros_like(a)
    split.prefill_attn_paged(b, w.q, w.gate, lay, torch.from_numpy(w.owner.astype(np.int32)).cuda(), w.dlen, window)
    torch.cuda.synchronize()
    assert split.device_status() == 0
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))


def test_repeated_launches_and_graph_replay(kvs):
    """The unit tables and the partial slots are rewritten by every launch: back-to-back launches of
    different waves and a captured graph give the same bits as single launches."""
    import torch
    split, _ = kvs
    w1, w2 = Wave([(7000, 64)], seed=31), Wave([(900, 200), (3000, 10)], seed=32)
    a1, a2 = w1.run(split, 0), w2.run(split, 0)
    for _ in range(3):
        b1, b2 = w1.run(split, 0), w2.run(split, 0)
        assert torch.equal(a1.view(torch.int16), b1.view(torch.int16))
        assert torch.equal(a2.view(torch.int16), b2.view(torch.int16))
    ctx = torch.zeros_like(a1)
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        split.prefill_attn(ctx, w1.q, w1.gate, w1.kp, w1.vp, w1.dlen, 0)  # warm-up on the capture stream
        s.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            split.prefill_attn(ctx, w1.q, w1.gate, w1.kp, w1.vp, w1.dlen, 0)
        ctx.zero_()
        g.replay()
        g.replay()
    s.synchronize()
    torch.cuda.synchronize()
    assert torch.equal(ctx.view(torch.int16), a1.view(torch.int16))
