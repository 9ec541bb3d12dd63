"""The paged K/V entry points through the C ABI: the same keys stored in blocks of a pool behind
block tables must give results that are bit-identical to the contiguous pointer-table entry points
(the work items are the same 256-key ranges in the same order), and the appended rows must land
in the right slot of the right block."""
import numpy as np
import pytest

from oracle import cpu as O
from tests.kvcase import DecodeCase, NKV, HD

pytestmark = pytest.mark.gpu

LENS = [0, 1, 14, 15, 16, 17, 255, 256, 257, 1000, 2047, 4095]


@pytest.fixture(scope="module")
def kv():
    from oxide_infer_b200 import KvPath
    return KvPath(0, max_batch=64, max_seq_len=8192, max_prefill_rows=0)


def _paged(case, d, block_size, seed, layers_in_block=1, layer=0):
    """Scatters the case's contiguous device caches into blocks of one pool.  With layers_in_block > 1
    the pool has the reference's shape (paged_pool.rs:20-24): every block holds K and V of all
    layers, so the block stride is 2 * layers * block_size rows and the layer's K / V rows start
    inside the block."""
    import torch
    from oxide_infer_b200 import PagedLayout
    rng = np.random.default_rng(seed)
    need = [(int(n) + 1 + block_size - 1) // block_size for n in case.lens]  # blocks incl. the appended token
    total = sum(need) + 3
    perm = rng.permutation(total).astype(np.int32)
    max_blocks = max(need) + 1
    tables = np.full((case.b, max_blocks), 0, np.int32)
    rows_per_block = 2 * layers_in_block * block_size
    pool = torch.zeros(total, rows_per_block, NKV, HD, dtype=torch.float16, device="cuda")
    k_view = pool[:, (2 * layer) * block_size:(2 * layer + 1) * block_size]
    v_view = pool[:, (2 * layer + 1) * block_size:(2 * layer + 2) * block_size]
    o = 0
    for i, n in enumerate(case.lens):
        ids = perm[o:o + need[i]]
        o += need[i]
        tables[i, :need[i]] = ids
        for j, bid in enumerate(ids):
            lo, hi = j * block_size, min((j + 1) * block_size, int(n))
            if hi > lo:
                k_view[bid, :hi - lo] = d.k_cache[i][lo:hi]
                v_view[bid, :hi - lo] = d.v_cache[i][lo:hi]
    dt = torch.from_numpy(tables).cuda()
    lay = PagedLayout.of(k_view, v_view, dt, block_size, block_stride_bytes=rows_per_block * NKV * HD * 2, num_blocks=total)
    return lay, pool, k_view, v_view, tables


@pytest.mark.parametrize("block_size", [16, 64, 256])
@pytest.mark.parametrize("window", [0, 300])
def test_paged_append_then_attention_equals_contiguous(kv, block_size, window):
    import torch
    case = DecodeCase(LENS, seed=41)
    d = case.device()
    lay, pool, k_view, v_view, tables = _paged(case, d, block_size, seed=42)
    # contiguous path
    kv.append(d.q, d.k, d.v, d.q_norm_w, d.k_norm_w, d.cos, d.sin, d.pos_ids, d.k_ptrs, d.v_ptrs)
    kv.decode_attn(d.ctx, d.q, d.gate, d.k_ptrs, d.v_ptrs, d.seq_lens, window)
    # paged path on fresh inputs
    d2 = case.device()
    kv.append_paged(d2.q, d2.k, d2.v, d2.q_norm_w, d2.k_norm_w, d2.cos, d2.sin, d2.pos_ids, lay)
    kv.decode_attn_paged(d2.ctx, d2.q, d2.gate, lay, d2.seq_lens, window)
    torch.cuda.synchronize()
    assert kv.device_status() == 0
    assert torch.equal(d.q, d2.q)
    for i, n in enumerate(case.lens):
        bid, slot = tables[i, int(n) // block_size], int(n) % block_size
        assert torch.equal(k_view[bid, slot], d.k_cache[i][int(n)]), i
        assert torch.equal(v_view[bid, slot], d.v_cache[i][int(n)]), i
    assert torch.equal(d.ctx.view(torch.int16), d2.ctx.view(torch.int16))
    # and against the oracle on the contiguous copy
    h = case.host()
    O.qk_rmsnorm(h.q, case.q_norm_w)
    O.qk_rmsnorm(h.k, case.k_norm_w)
    O.rope(h.q, case.cos, case.sin, case.pos_ids)
    O.rope(h.k, case.cos, case.sin, case.pos_ids)
    O.kv_copy(h.k_ptrs, h.k, case.pos_ids)
    O.kv_copy(h.v_ptrs, h.v, case.pos_ids)
    want = O.decode_attn(h.q, case.gate, h.k_ptrs, h.v_ptrs, case.seq_lens, window)
    err = np.abs(d2.ctx.cpu().numpy().astype(np.float32) - want.astype(np.float32)).max()
    assert err <= 2e-3, err


@pytest.mark.parametrize("block_size", [16, 128])
def test_paged_fused_step_equals_contiguous_fused_step(kv, block_size):
    import torch
    case = DecodeCase(LENS, seed=43)
    d = case.device()
    kv.append_decode(d.ctx, d.q, d.k, d.v, d.gate, d.q_norm_w, d.k_norm_w, d.cos, d.sin, d.pos_ids, d.seq_lens,
                     d.k_ptrs, d.v_ptrs, 0)
    d2 = case.device()
    lay, pool, k_view, v_view, tables = _paged(case, d2, block_size, seed=44)
    kv.append_decode_paged(d2.ctx, d2.q, d2.k, d2.v, d2.gate, d2.q_norm_w, d2.k_norm_w, d2.cos, d2.sin, d2.seq_lens, lay, 0)
    torch.cuda.synchronize()
    assert kv.device_status() == 0
    assert torch.equal(d.ctx.view(torch.int16), d2.ctx.view(torch.int16))
    for i, n in enumerate(case.lens):
        bid, slot = tables[i, int(n) // block_size], int(n) % block_size
        assert torch.equal(k_view[bid, slot], d.k_cache[i][int(n)]), i
        assert torch.equal(v_view[bid, slot], d.v_cache[i][int(n)]), i


def test_paged_reference_pool_shape(kv):
    """Blocks that hold K and V of 3 layers (block stride = 6 * block_size rows), layer 1 addressed."""
    import torch
    case = DecodeCase([100, 700, 31], seed=45)
    d = case.device()
    kv.append(d.q, d.k, d.v, d.q_norm_w, d.k_norm_w, d.cos, d.sin, d.pos_ids, d.k_ptrs, d.v_ptrs)
    kv.decode_attn(d.ctx, d.q, d.gate, d.k_ptrs, d.v_ptrs, d.seq_lens, 0)
    d2 = case.device()
    lay, pool, k_view, v_view, tables = _paged(case, d2, 16, seed=46, layers_in_block=3, layer=1)
    before = pool.clone()
    kv.append_paged(d2.q, d2.k, d2.v, d2.q_norm_w, d2.k_norm_w, d2.cos, d2.sin, d2.pos_ids, lay)
    kv.decode_attn_paged(d2.ctx, d2.q, d2.gate, lay, d2.seq_lens, 0)
    torch.cuda.synchronize()
    assert torch.equal(d.ctx.view(torch.int16), d2.ctx.view(torch.int16))
    changed = (pool != before).any(dim=(2, 3))  # [block][row in block]
    assert int(changed.sum()) <= 2 * case.b     # only the appended K and V rows
    assert not changed[:, :32].any() and not changed[:, 64:].any()  # layers 0 and 2 untouched


def test_paged_bad_tables_are_flagged_not_followed(kv):
    import torch
    from oxide_infer_b200 import OxiError, PagedLayout
    case = DecodeCase([40, 90], seed=47)
    d = case.device()
    lay, pool, k_view, v_view, tables = _paged(case, d, 16, seed=48)
    bad = tables.copy()
    bad[1, 2] = 10 ** 6  # beyond the pool
    dt = torch.from_numpy(bad).cuda()
    lay_bad = PagedLayout.of(k_view, v_view, dt, 16, block_stride_bytes=lay.block_stride_bytes, num_blocks=lay.num_blocks)
    kv.decode_attn_paged(d.ctx, d.q, d.gate, lay_bad, d.seq_lens, 0)
    torch.cuda.synchronize()
    assert kv.device_status() & 16  # OXI_DEV_BAD_BLOCK
    # a table with too few columns for the row: flagged, row skipped
    short = torch.from_numpy(np.ascontiguousarray(tables[:, :3])).cuda()
    lay_short = PagedLayout.of(k_view, v_view, short, 16, block_stride_bytes=lay.block_stride_bytes, num_blocks=lay.num_blocks)
    d.ctx.fill_(7.0)
    kv.decode_attn_paged(d.ctx, d.q, d.gate, lay_short, d.seq_lens, 0)
    torch.cuda.synchronize()
    assert kv.device_status() & 2   # OXI_DEV_BAD_SEQ_LEN
    assert bool((d.ctx[1] == 7.0).all())  # 91 keys need 6 blocks, the table has 3 columns
    # host-side validation
    with pytest.raises(OxiError):
        kv.decode_attn_paged(d.ctx, d.q, d.gate, PagedLayout.of(k_view, v_view, dt, 8, block_stride_bytes=lay.block_stride_bytes), d.seq_lens, 0)
    with pytest.raises(OxiError):
        kv.decode_attn_paged(d.ctx, d.q, d.gate, PagedLayout.of(k_view, v_view, dt, 16, block_stride_bytes=1000), d.seq_lens, 0)


@pytest.mark.parametrize("block_size,window", [(16, 0), (64, 0), (16, 200), (256, 0)])
def test_paged_prefill_equals_contiguous_prefill(block_size, window):
    """A wave of chunks (ragged lengths, prefixes that are not multiples of anything) over paged
    caches: ctx must be bit-identical to oxi_prefill_attn over contiguous copies of the same keys."""
    import torch
    from oxide_infer_b200 import KvPath, PagedLayout
    rng = np.random.default_rng(61)
    chunks = [(0, 70), (333, 128), (1000, 1), (77, 64), (2049, 129)]  # (prefix, new rows)
    rows = sum(n for _, n in chunks)
    kvp = KvPath(0, max_batch=8, max_seq_len=4096, max_prefill_rows=rows)
    g = torch.Generator(device="cuda").manual_seed(61)
    rn = lambda *s: torch.empty(*s, dtype=torch.float16, device="cuda").normal_(generator=g)
    kc = [rn(p + n, NKV, HD) for p, n in chunks]
    vc = [rn(p + n, NKV, HD) for p, n in chunks]
    q, gate = rn(rows, 16, HD), rn(rows, 16)
    owner = np.concatenate([np.full(n, i) for i, (_, n) in enumerate(chunks)])
    lens = np.concatenate([p + 1 + np.arange(n) for p, n in chunks]).astype(np.int32)
    kp = torch.tensor([kc[i].data_ptr() for i in owner], dtype=torch.int64, device="cuda")
    vp = torch.tensor([vc[i].data_ptr() for i in owner], dtype=torch.int64, device="cuda")
    dlen = torch.from_numpy(lens).cuda()
    ctx = torch.zeros(rows, 16, HD, dtype=torch.float16, device="cuda")
    kvp.prefill_attn(ctx, q, gate, kp, vp, dlen, window)
    # the same keys in scattered blocks
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
            kpool[bid, :hi - lo] = kc[i][lo:hi]
            vpool[bid, :hi - lo] = vc[i][lo:hi]
    lay = PagedLayout.of(kpool, vpool, torch.from_numpy(tables).cuda(), block_size)
    ctx2 = torch.zeros_like(ctx)
    kvp.prefill_attn_paged(ctx2, q, gate, lay, torch.from_numpy(owner.astype(np.int32)).cuda(), dlen, window)
    torch.cuda.synchronize()
    assert kvp.device_status() == 0
    assert torch.equal(ctx.view(torch.int16), ctx2.view(torch.int16))


@pytest.mark.parametrize("block_size,window", [(32, 77), (16, 1024)])
def test_paged_fused_step_with_window(kv, block_size, window):
    """Sliding windows start in the middle of a block and of a 4-token copy group."""
    import torch
    case = DecodeCase([5, 76, 77, 78, 300, 1023, 1024, 1025, 3000], seed=49)
    d = case.device()
    kv.append_decode(d.ctx, d.q, d.k, d.v, d.gate, d.q_norm_w, d.k_norm_w, d.cos, d.sin, d.pos_ids, d.seq_lens,
                     d.k_ptrs, d.v_ptrs, window)
    d2 = case.device()
    lay, pool, k_view, v_view, tables = _paged(case, d2, block_size, seed=50)
    kv.append_decode_paged(d2.ctx, d2.q, d2.k, d2.v, d2.gate, d2.q_norm_w, d2.k_norm_w, d2.cos, d2.sin, d2.seq_lens, lay,
                           window)
    torch.cuda.synchronize()
    assert kv.device_status() == 0
    assert torch.equal(d.ctx.view(torch.int16), d2.ctx.view(torch.int16))


def test_paged_decode_with_shared_prefix_blocks(kv):
    """Two sequences whose tables point at the same physical blocks for a common 64-token prefix (what the
    block manager's reference counts are for): each gets the result of its own contiguous copy."""
    import torch
    from oxide_infer_b200 import PagedLayout
    bs, shared_tokens = 16, 64
    case = DecodeCase([200, 333], seed=77)
    d = case.device()
    # make the prefix common in the contiguous caches too
    d.k_cache[1][:shared_tokens] = d.k_cache[0][:shared_tokens]
    d.v_cache[1][:shared_tokens] = d.v_cache[0][:shared_tokens]
    kv.append(d.q, d.k, d.v, d.q_norm_w, d.k_norm_w, d.cos, d.sin, d.pos_ids, d.k_ptrs, d.v_ptrs)
    kv.decode_attn(d.ctx, d.q, d.gate, d.k_ptrs, d.v_ptrs, d.seq_lens, 0)
    need = [(int(n) + 1 + bs - 1) // bs for n in case.lens]
    nshared = shared_tokens // bs
    total = need[0] + need[1] - nshared + 1
    kpool = torch.zeros(total, bs, NKV, HD, dtype=torch.float16, device="cuda")
    vpool = torch.zeros_like(kpool)
    tables = np.zeros((2, max(need)), np.int32)
    tables[0, :need[0]] = np.arange(1, need[0] + 1)
    tables[1, :nshared] = tables[0, :nshared]  # the shared blocks
    tables[1, nshared:need[1]] = np.arange(need[0] + 1, need[0] + 1 + need[1] - nshared)
    for i in range(2):
        for j in range(need[i]):
            lo, hi = j * bs, min((j + 1) * bs, int(case.lens[i]) + 1)
            kpool[tables[i, j], :hi - lo] = d.k_cache[i][lo:hi]
            vpool[tables[i, j], :hi - lo] = d.v_cache[i][lo:hi]
    lay = PagedLayout.of(kpool, vpool, torch.from_numpy(tables).cuda(), bs)
    ctx = torch.zeros_like(d.ctx)
    kv.decode_attn_paged(ctx, d.q, d.gate, lay, d.seq_lens, 0)
    torch.cuda.synchronize()
    assert kv.device_status() == 0
    assert torch.equal(ctx.view(torch.int16), d.ctx.view(torch.int16))
