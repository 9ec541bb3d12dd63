"""oxi_prefill_attn against the reference's GEMM prefill path: its pack_q / softmax_mask / gate_scatter
kernels with float32 matmuls in place of the two cuBLASLt calls (batch_engine.rs:439-592), on the
reference's own chunk shapes - both live on this GPU and through the committed fixture
tests/golden/ref_gemm_prefill_b200.npz."""
import importlib.util
import os

import numpy as np
import pytest
import torch

from tests.kvcase import NQ, HD, u32

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
_spec = importlib.util.spec_from_file_location("make_ref_gemm_prefill_golden",
                                               os.path.join(HERE, "golden", "make_ref_gemm_prefill_golden.py"))
GP = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(GP)

ATTN_TOL = 2e-3


@pytest.fixture(scope="module")
def kv():
    from oxide_infer_b200 import KvPath, build
    build.build()
    p = KvPath(0, max_batch=8, max_seq_len=1024, max_prefill_rows=256)
    yield p
    assert p.device_status() == 0
    p.close()


def _ours(kv, x, rows, p0, window):
    d = {k: torch.from_numpy(v).cuda() for k, v in x.items()}
    kp = torch.full((rows,), d["k"].data_ptr(), dtype=torch.int64, device="cuda")
    vp = torch.full((rows,), d["v"].data_ptr(), dtype=torch.int64, device="cuda")
    sl = u32(np.arange(p0 + 1, p0 + rows + 1, dtype=np.uint32))
    ctx = torch.zeros(rows, NQ, HD, dtype=torch.float16, device="cuda")
    kv.prefill_attn(ctx, d["q"], d["gate"], kp, vp, sl, window)
    torch.cuda.synchronize()
    return d, sl, ctx


@pytest.mark.parametrize("rows,p0,window", GP.CASES)
def test_prefill_attn_matches_reference_gemm_path_fixture(kv, rows, p0, window):
    gold = np.load(os.path.join(HERE, "golden", "ref_gemm_prefill_b200.npz"))
    _, _, ctx = _ours(kv, GP.chunk_inputs(rows, p0), rows, p0, window)
    got = ctx.cpu().numpy()[GP.keep_rows(rows)].astype(np.float32)
    want = gold["ctx_" + GP.case_name(rows, p0, window)].astype(np.float32)
    assert np.abs(got - want).max() <= ATTN_TOL


@pytest.mark.parametrize("rows,p0,window", GP.CASES)
def test_prefill_attn_matches_reference_gemm_path_live(kv, ref, rows, p0, window):
    if ref is None:
        pytest.skip("oracle-only run requested")
    gold = np.load(os.path.join(HERE, "golden", "ref_gemm_prefill_b200.npz"))
    d, sl, ctx = _ours(kv, GP.chunk_inputs(rows, p0), rows, p0, window)
    rctx = torch.zeros_like(ctx)
    sums = ref.gemm_attention_chunk(rctx, d["q"], d["gate"], d["k"], d["v"], sl, rows, p0 + 1, p0 + rows, window)
    torch.cuda.synchronize()
    assert np.abs(ctx.float().cpu().numpy() - rctx.float().cpu().numpy()).max() <= ATTN_TOL
    # the live run reproduces the committed fixture (same kernels, same GPU type, float32 matmuls)
    keep = GP.keep_rows(rows)
    want = gold["ctx_" + GP.case_name(rows, p0, window)].astype(np.float32)
    assert np.abs(rctx.cpu().numpy()[keep].astype(np.float32) - want).max() <= 5e-4
    assert np.allclose(sums.cpu().numpy(), gold["sums_" + GP.case_name(rows, p0, window)], rtol=1e-5)
