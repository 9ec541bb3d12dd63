"""Stream ordering of consecutive decode steps (batch_engine.rs:689-691, 709-740: the engine
rebuilds positions and lengths for every token and enqueues step after step on one stream).

Every test runs 12 consecutive tokens through three attention layers WITHOUT a host
synchronisation between the steps and requires caches, positions and contexts to be the bytes
of 12 steps whose tables were built on the host and uploaded before each step:
  * the host-buffer entry, steps enqueued back to back (pinned and pageable memory);
  * a captured graph of the host-buffer entry, replayed with new positions in the same pinned
    buffer;
  * the device-table form: (fused step of every layer, oxi_advance_step) x 12, eagerly on one
    stream."""
import numpy as np
import pytest
import torch

from tests.kvcase import NQ, HD, DecodeCase, u32

pytestmark = pytest.mark.gpu

STEPS, LAYERS = 12, 3
LENS = [5, 250, 251, 1020, 31, 767]


@pytest.fixture(scope="module")
def kv():
    from oxide_infer_b200 import KvPath, build
    build.build()
    p = KvPath(0, max_batch=8, max_seq_len=2048, max_prefill_rows=0)
    yield p
    assert p.device_status() == 0
    p.close()


def _case():
    return DecodeCase(LENS, seed=71, spare_rows=STEPS + 1, max_pos=max(LENS) + STEPS + 2)


def _host_table_steps(kv, case):
    """The yardstick: tables built on the host for every step, uploaded before the step."""
    de = [case.device() for _ in range(LAYERS)]
    ctxs = []
    for s in range(STEPS):
        pos, sl = u32(case.lens + s), u32(case.lens + s + 1)
        for d in de:
            kv.append_decode(d.ctx, d.q, d.k, d.v, d.gate, d.q_norm_w, d.k_norm_w, d.cos, d.sin, pos, sl,
                             d.k_ptrs, d.v_ptrs, 0)
        torch.cuda.synchronize()
        ctxs.append(torch.stack([d.ctx for d in de]).cpu())
    return de, ctxs


def _same_caches(de, dg):
    for l in range(LAYERS):
        for i in range(len(LENS)):
            assert torch.equal(de[l].k_cache[i].view(torch.int16), dg[l].k_cache[i].view(torch.int16)), (l, i)
            assert torch.equal(de[l].v_cache[i].view(torch.int16), dg[l].v_cache[i].view(torch.int16)), (l, i)


def _host_inputs(dg, place):
    stack = lambda name: place(torch.stack([getattr(d, name) for d in dg]))
    qw = torch.stack([d.q_norm_w for d in dg]).contiguous()
    kw = torch.stack([d.k_norm_w for d in dg]).contiguous()
    return stack("q"), stack("k"), stack("v"), stack("gate"), stack("k_ptrs"), stack("v_ptrs"), qw, kw


@pytest.mark.parametrize("pinned", [True, False])
def test_host_buffer_steps_back_to_back_without_sync(kv, pinned):
    case = _case()
    b = len(LENS)
    de, want = _host_table_steps(kv, case)
    dg = [case.device() for _ in range(LAYERS)]
    place = (lambda t: t.cpu().pin_memory()) if pinned else (lambda t: t.cpu())
    hq, hk, hv, hg, hkp, hvp, qw, kw = _host_inputs(dg, place)
    # one position row and one context block per step: the caller may not touch a buffer of an
    # enqueued step before that step has run, but it may enqueue the next one
    hpos = torch.from_numpy(np.stack([(case.lens + s).astype(np.uint32).view(np.int32) for s in range(STEPS)]))
    hctx = torch.zeros(STEPS, LAYERS, b, NQ, HD, dtype=torch.float16)
    if pinned:
        hpos, hctx = hpos.pin_memory(), hctx.pin_memory()
    for s in range(STEPS):
        kv.decode_step_host(hctx[s], hq, hk, hv, hg, qw, kw, dg[0].cos, dg[0].sin, hpos[s], hkp, hvp, b, LAYERS)
    torch.cuda.synchronize()
    for s in range(STEPS):
        assert torch.equal(hctx[s].view(torch.int16), want[s].view(torch.int16)), s
    _same_caches(de, dg)


def test_host_buffer_graph_replays_with_new_positions(kv):
    case = _case()
    b = len(LENS)
    de, want = _host_table_steps(kv, case)
    dg = [case.device() for _ in range(LAYERS)]
    pin = lambda t: t.cpu().pin_memory()
    hq, hk, hv, hg, hkp, hvp, qw, kw = _host_inputs(dg, pin)
    hpos = torch.from_numpy(case.lens.astype(np.uint32).view(np.int32).copy()).pin_memory()
    hctx = torch.zeros(LAYERS, b, NQ, HD, dtype=torch.float16).pin_memory()
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            kv.decode_step_host(hctx, hq, hk, hv, hg, qw, kw, dg[0].cos, dg[0].sin, hpos, hkp, hvp, b, LAYERS)
        for s in range(STEPS):
            hpos.copy_(torch.from_numpy((case.lens + s).astype(np.uint32).view(np.int32)))
            graph.replay()
            side.synchronize()  # the replay reads hpos and writes hctx: finish before the host touches them
            assert torch.equal(hctx.view(torch.int16), want[s].view(torch.int16)), s
    _same_caches(de, dg)


def test_device_tables_advance_eagerly_between_steps(kv):
    case = _case()
    de, want = _host_table_steps(kv, case)
    dg = [case.device() for _ in range(LAYERS)]
    pos, sl = u32(case.lens.copy()), u32(case.lens + 1)
    ctxs = torch.zeros(STEPS, LAYERS, len(LENS), NQ, HD, dtype=torch.float16, device="cuda")
    torch.cuda.synchronize()
    for s in range(STEPS):
        for l, d in enumerate(dg):
            kv.append_decode(ctxs[s, l], d.q, d.k, d.v, d.gate, d.q_norm_w, d.k_norm_w, d.cos, d.sin, pos, sl,
                             d.k_ptrs, d.v_ptrs, 0)
        kv.advance_step(pos, sl, 1)
    torch.cuda.synchronize()
    assert np.array_equal(pos.cpu().numpy().view(np.uint32), case.lens + STEPS)
    assert np.array_equal(sl.cpu().numpy().view(np.uint32), case.lens + STEPS + 1)
    for s in range(STEPS):
        assert torch.equal(ctxs[s].cpu().view(torch.int16), want[s].view(torch.int16)), s
    _same_caches(de, dg)


def test_host_buffer_step_with_more_layers_than_staging_sets(kv):
    """Nineteen layers: the host-buffer entry stages a group of sixteen layers at a time (eight on handles of more than
    256 rows), so layers 16-18 reuse the staging of layers 0-2 (their uploads wait for the first group's kernels, their
    kernels for its downloads).  Two steps back to back."""
    layers, b = 19, len(LENS)
    cases = [DecodeCase(LENS, seed=200 + l, spare_rows=3, max_pos=max(LENS) + 4) for l in range(layers)]
    dev = [c.device() for c in cases]
    hst = [c.device() for c in cases]
    want = []
    for s in range(2):
        pos, sl = u32(cases[0].lens + s), u32(cases[0].lens + s + 1)
        for d in dev:
            kv.append_decode(d.ctx, d.q, d.k, d.v, d.gate, d.q_norm_w, d.k_norm_w, d.cos, d.sin, pos, sl, d.k_ptrs, d.v_ptrs, 0)
        torch.cuda.synchronize()
        want.append(torch.stack([d.ctx for d in dev]).cpu())
    pin = lambda t: t.cpu().pin_memory()
    stack = lambda name: pin(torch.stack([getattr(d, name) for d in hst]))
    hq, hk, hv, hg, hkp, hvp = stack("q"), stack("k"), stack("v"), stack("gate"), stack("k_ptrs"), stack("v_ptrs")
    qw = torch.stack([d.q_norm_w for d in hst]).contiguous()
    kw = torch.stack([d.k_norm_w for d in hst]).contiguous()
    hpos = torch.from_numpy(np.stack([(cases[0].lens + s).astype(np.uint32).view(np.int32) for s in range(2)])).pin_memory()
    hctx = torch.zeros(2, layers, b, NQ, HD, dtype=torch.float16).pin_memory()
    for s in range(2):
        kv.decode_step_host(hctx[s], hq, hk, hv, hg, qw, kw, hst[0].cos, hst[0].sin, hpos[s], hkp, hvp, b, layers)
    torch.cuda.synchronize()
    for s in range(2):
        assert torch.equal(hctx[s].view(torch.int16), want[s].view(torch.int16)), s
    for l in range(layers):
        for i in range(b):
            assert torch.equal(hst[l].k_cache[i].view(torch.int16), dev[l].k_cache[i].view(torch.int16)), (l, i)
