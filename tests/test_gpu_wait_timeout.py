"""The bounded in-kernel waits run out, on purpose and without a fault.

Every pipeline wait of the streaming kernels (decode: consumers waiting for a stage of K/V rows;
prefill: tensor-core warps waiting for a K tile) gives up after a limit, the CTA finishes without
output and OXI_DEV_WAIT_TIMEOUT is raised.  oxi_debug_arm_wait_fault makes CTA 0 of the next launch
withhold one stage and shortens the limit to a millisecond, so that path executes: the call
returns, the status bit is set, rows that CTA 0 did not own are correct, and the handle's next
launch is bit-identical to a launch on a fresh handle."""
import numpy as np
import pytest
import torch

from tests.kvcase import NQ, NKV, HD, DecodeCase, dev_ptr_table, u32

pytestmark = pytest.mark.gpu

WAIT_TIMEOUT = 4


@pytest.fixture()
def kv():
    from oxide_infer_b200 import KvPath, build
    build.build()
    p = KvPath(0, max_batch=64, max_seq_len=8192, max_prefill_rows=512)
    yield p
    p.close()


@pytest.mark.parametrize("fused", [False, True])
@pytest.mark.parametrize("stage", [0, 4])
def test_decode_wait_runs_out_and_the_handle_recovers(kv, fused, stage):
    lens = [2000, 300, 4095, 64, 1500, 700]  # row 0 -> CTA 0's first item has 8 stages of 32 keys
    case = DecodeCase(lens, seed=90)

    def run(d):
        if fused:
            kv.append_decode(d.ctx, d.q, d.k, d.v, d.gate, d.q_norm_w, d.k_norm_w, d.cos, d.sin, d.pos_ids, d.seq_lens,
                             d.k_ptrs, d.v_ptrs, 0)
        else:
            kv.append(d.q, d.k, d.v, d.q_norm_w, d.k_norm_w, d.cos, d.sin, d.pos_ids, d.k_ptrs, d.v_ptrs)
            kv.decode_attn(d.ctx, d.q, d.gate, d.k_ptrs, d.v_ptrs, d.seq_lens, 0)

    good = case.device()
    run(good)
    torch.cuda.synchronize()
    assert kv.device_status() == 0

    hit = case.device()
    kv.arm_wait_fault(0, stage, 1000)
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    run(hit)
    t1.record()
    torch.cuda.synchronize()                       # the launch returns: no hang
    assert t0.elapsed_time(t1) < 500.0             # milliseconds, not the one-second production limit
    assert kv.device_status() == WAIT_TIMEOUT      # reported, and cleared by the read
    assert kv.device_status() == 0
    # CTA 0 took work item 0 = (row 0, first key range); rows it did not touch are right
    assert torch.equal(hit.ctx[1].view(torch.int16), good.ctx[1].view(torch.int16))
    assert torch.equal(hit.ctx[3].view(torch.int16), good.ctx[3].view(torch.int16))

    again = case.device()                          # the fault was armed for one launch only
    run(again)
    torch.cuda.synchronize()
    assert kv.device_status() == 0
    assert torch.equal(again.ctx.view(torch.int16), good.ctx.view(torch.int16))
    for i in range(case.b):
        assert torch.equal(again.k_cache[i].view(torch.int16), good.k_cache[i].view(torch.int16))


@pytest.mark.parametrize("tile", [0, 5])
def test_prefill_wait_runs_out_and_the_handle_recovers(kv, tile):
    rng = np.random.default_rng(91)
    nseq, n = 3, 128
    prefix = [1000, 900, 600]  # every (64-row block, KV head) item scans at least 11 K tiles
    caches, kp, vp, sl = [], [], [], []
    for p0 in prefix:
        k = torch.from_numpy(rng.standard_normal((p0 + n, NKV, HD), dtype=np.float32).astype(np.float16)).cuda()
        v = torch.from_numpy(rng.standard_normal((p0 + n, NKV, HD), dtype=np.float32).astype(np.float16)).cuda()
        caches.append((k, v))
        kp += [k.data_ptr()] * n
        vp += [v.data_ptr()] * n
        sl += [p0 + r + 1 for r in range(n)]
    rows = nseq * n
    q = torch.from_numpy(rng.standard_normal((rows, NQ, HD), dtype=np.float32).astype(np.float16)).cuda()
    gate = torch.from_numpy(rng.standard_normal((rows, NQ), dtype=np.float32).astype(np.float16)).cuda()
    kpt = torch.tensor(kp, dtype=torch.int64, device="cuda")
    vpt = torch.tensor(vp, dtype=torch.int64, device="cuda")
    slt = u32(np.asarray(sl, np.uint32))
    kv.prefill_split_configure(0, 0)  # unsplit: 6 blocks x 4 KV heads = 24 items, CTA 0 takes the longest

    def run():
        ctx = torch.zeros(rows, NQ, HD, dtype=torch.float16, device="cuda")
        kv.prefill_attn(ctx, q, gate, kpt, vpt, slt, 0)
        torch.cuda.synchronize()
        return ctx

    good = run()
    assert kv.device_status() == 0
    kv.arm_wait_fault(1, tile, 1000)
    hit = run()
    assert kv.device_status() == WAIT_TIMEOUT
    assert kv.device_status() == 0
    # CTA 0 wrote nothing for its item (64 rows of one KV head stay zero); everything written is right
    written = hit.view(rows, NKV, 4 * HD).abs().sum(-1) > 0
    assert not written.all() and written.any()
    assert torch.equal(hit.view(rows, NKV, 4 * HD)[written], good.view(rows, NKV, 4 * HD)[written])
    again = run()
    assert kv.device_status() == 0
    assert torch.equal(again.view(torch.int16), good.view(torch.int16))


@pytest.mark.parametrize("rows,stage", [(128, 0), (128, 6), (600, 0), (600, 9)])
def test_projection_wait_runs_out_and_the_handle_recovers(rows, stage):
    """The projection GEMMs: 128 rows run the four-CTA cluster kernel (CTA 0 = the first quarter of k of head 0's tile),
    600 rows the CTA-pair kernel (CTA 0 = the leader of the pair that owns rows 0-255 of q heads 0 and 1).  The armed launch
    returns within milliseconds with the status bit set, every tile of another cluster is right, nothing of the
    cluster's own tile is written, and the next launch is bit-identical to an undisturbed one."""
    from oxide_infer_b200 import KvPath, Linear, build
    build.build()
    kv = KvPath(0, max_batch=64, max_seq_len=2048, max_prefill_rows=1024)
    lens = [40 + (i % 300) for i in range(rows)]
    case = DecodeCase(lens, seed=93)
    g = torch.Generator(device="cuda").manual_seed(93)
    x = torch.randn(rows, 2048, device="cuda", generator=g).half()
    ws = [(torch.randn(o, 2048, device="cuda", generator=g) * 2048 ** -0.5).half() for o in (NQ * HD, NKV * HD, NKV * HD, NQ)]
    lin = Linear(*ws)

    def run(d, q_out, gate_out):
        kv.project_append(lin, x, q_out, gate_out, d.q_norm_w, d.k_norm_w, d.cos, d.sin, d.pos_ids, d.k_ptrs, d.v_ptrs)

    new_out = lambda: (torch.full((rows, NQ, HD), 7.0, dtype=torch.float16, device="cuda"),
                       torch.zeros(rows, NQ, dtype=torch.float16, device="cuda"))
    good, (gq, gg) = case.device(), new_out()
    run(good, gq, gg)
    torch.cuda.synchronize()
    assert kv.device_status() == 0

    hit, (hq, hg) = case.device(), new_out()
    kv.arm_wait_fault(2, stage, 1000)
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    run(hit, hq, hg)
    t1.record()
    torch.cuda.synchronize()                       # the launch returns: no hang
    assert t0.elapsed_time(t1) < 500.0
    assert kv.device_status() == WAIT_TIMEOUT
    assert kv.device_status() == 0
    own_heads = 1 if rows <= 512 else 2            # the tile of CTA 0's cluster: head 0 (and 1) of the first 128 (256) rows
    own_rows = min(rows, 128 if rows <= 512 else 256)
    assert torch.equal(hq[:, own_heads:].contiguous().view(torch.int16), gq[:, own_heads:].contiguous().view(torch.int16))
    assert torch.equal(hq[own_rows:].view(torch.int16), gq[own_rows:].view(torch.int16))
    assert bool((hq[:own_rows, :own_heads] == 7.0).all())          # nothing written where the cluster gave up
    assert torch.equal(hg.view(torch.int16), gg.view(torch.int16))
    for i in range(rows):
        assert torch.equal(hit.k_cache[i].view(torch.int16), good.k_cache[i].view(torch.int16)), i
        assert torch.equal(hit.v_cache[i].view(torch.int16), good.v_cache[i].view(torch.int16)), i

    again, (aq, ag) = case.device(), new_out()     # armed for one launch only
    run(again, aq, ag)
    torch.cuda.synchronize()
    assert kv.device_status() == 0
    assert torch.equal(aq.view(torch.int16), gq.view(torch.int16))
    for i in (0, rows // 2, rows - 1):
        assert torch.equal(again.k_cache[i].view(torch.int16), good.k_cache[i].view(torch.int16))
    kv.close()
