"""oxi_argmax / oxi_embed_lookup through the C ABI against the CPU oracle, the reference's own
kernels (when their cubins are present) and the committed golden outputs: token ids and gathered
bytes must be identical."""
import importlib.util
import os

import numpy as np
import pytest

from oracle import cpu as O

HERE = os.path.dirname(os.path.abspath(__file__))
spec = importlib.util.spec_from_file_location("make_ref_sample_golden", os.path.join(HERE, "golden", "make_ref_sample_golden.py"))
G = importlib.util.module_from_spec(spec)
spec.loader.exec_module(G)

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def kv():
    from oxide_infer_b200 import KvPath
    return KvPath(0, max_batch=256, max_seq_len=256, max_prefill_rows=0)


def _ours(kv, logits):
    import torch
    d = torch.from_numpy(logits).cuda()
    tok = torch.full((logits.shape[0],), -1, dtype=torch.int32, device="cuda")
    kv.argmax(tok, d)
    torch.cuda.synchronize()
    return tok.cpu().numpy().astype(np.uint32)


@pytest.mark.parametrize("name", list(G.sample_cases().keys()))
def test_argmax_cases(kv, name):
    logits = G.sample_cases()[name]
    got = _ours(kv, logits)
    assert np.array_equal(got, O.argmax(logits)), name
    gold = np.load(os.path.join(HERE, "golden", "ref_sample_b200.npz"))
    assert np.array_equal(got, gold["argmax_" + name]), name
    assert kv.device_status() == 0


def test_argmax_against_reference_kernel_live(kv):
    import torch
    from oracle import refptx
    if not refptx.available():
        pytest.skip("reference cubins not built")
    ref = refptx.RefPtx()
    rng = np.random.default_rng(31)
    for batch, vocab, q in [(1, 128000, 0.0), (5, 128000, 4.0), (130, 32000, 2.0), (256, 1000, 1.0), (3, 257, 8.0), (2, 7, 0.0)]:
        x = rng.standard_normal((batch, vocab), dtype=np.float32)
        if q:
            x = np.round(x * q) / q  # ties
        logits = x.astype(np.float16)
        d = torch.from_numpy(logits).cuda()
        rt = torch.zeros(batch, dtype=torch.int32, device="cuda")
        ref.argmax(rt, d, vocab, batch)
        torch.cuda.synchronize()
        got = _ours(kv, logits)
        assert np.array_equal(got, rt.cpu().numpy().astype(np.uint32)), (batch, vocab, q)
        assert np.array_equal(got, O.argmax(logits)), (batch, vocab, q)


def test_argmax_twice_and_full_batch(kv):
    """The arrival counters of the split rows are reset by the kernel itself: repeated launches
    and every split count (batch 1 ... 256 changes the CTAs per row) give the same tokens."""
    rng = np.random.default_rng(32)
    logits = (np.round(rng.standard_normal((256, 20000), dtype=np.float32) * 3) / 3).astype(np.float16)
    want = O.argmax(logits)
    for b in (256, 1, 3, 37, 148, 160, 230, 256):  # 160: two CTAs per row; 230: two would not be resident at once, so one
        assert np.array_equal(_ours(kv, logits[:b]), want[:b]), b


def test_embed_lookup(kv):
    import torch
    table, ids = G.embed_case()
    dt, di = torch.from_numpy(table).cuda(), torch.from_numpy(ids.astype(np.int32)).cuda()
    out = torch.zeros(ids.shape[0], table.shape[1], dtype=torch.float16, device="cuda")
    kv.embed_lookup(out, dt, di)
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    assert np.array_equal(got.view(np.uint16), O.embed_lookup(table, ids).view(np.uint16))
    gold = np.load(os.path.join(HERE, "golden", "ref_sample_b200.npz"))
    assert np.array_equal(got.view(np.uint16), gold["embed_rows"].view(np.uint16))
    assert kv.device_status() == 0


def test_embed_lookup_odd_hidden_and_bad_id(kv):
    import torch
    rng = np.random.default_rng(33)
    table = rng.standard_normal((40, 100), dtype=np.float32).astype(np.float16)  # 200-byte rows: scalar path
    ids = np.array([39, 0, 40, 12], np.uint32)  # 40 is beyond the table
    dt, di = torch.from_numpy(table).cuda(), torch.from_numpy(ids.astype(np.int32)).cuda()
    out = torch.full((4, 100), 7.0, dtype=torch.float16, device="cuda")
    kv.embed_lookup(out, dt, di)
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    assert np.array_equal(got[[0, 1, 3]], table[[39, 0, 12]])
    assert not got[2].any()
    assert kv.device_status() & 8  # OXI_DEV_BAD_TOKEN (reading the status clears it)


def test_argmax_unaligned_rows_and_tiny_vocabularies(kv):
    """Logits that do not start on a 16-byte boundary (scalar path) and vocabularies of 1 ... 9."""
    import torch
    rng = np.random.default_rng(34)
    for batch, vocab in [(3, 1), (2, 2), (4, 7), (2, 9), (5, 1003), (2, 128000)]:
        host = (np.round(rng.standard_normal(batch * vocab + 1, dtype=np.float32) * 2) / 2).astype(np.float16)
        flat = torch.from_numpy(host).cuda()
        logits = flat[1:].view(batch, vocab)  # data pointer is 2 bytes past a 16-byte boundary
        assert logits.data_ptr() % 16 == 2 and logits.is_contiguous()
        tok = torch.full((batch,), -1, dtype=torch.int32, device="cuda")
        kv.argmax(tok, logits)
        torch.cuda.synchronize()
        want = O.argmax(host[1:].reshape(batch, vocab))
        assert np.array_equal(tok.cpu().numpy().astype(np.uint32), want), (batch, vocab)


def test_advance_step_moves_only_what_it_is_given(kv):
    import torch
    pos = torch.arange(10, dtype=torch.int32, device="cuda")
    sl = pos + 1
    kv.advance_step(pos, sl, 3)
    kv.advance_step(None, sl, 2)
    kv.advance_step(pos, None, 0)
    torch.cuda.synchronize()
    assert torch.equal(pos.cpu(), torch.arange(10, dtype=torch.int32) + 3)
    assert torch.equal(sl.cpu(), torch.arange(10, dtype=torch.int32) + 6)
