"""The CPU oracle against outputs of the REFERENCE's own kernels run on a B200
(tests/golden/ref_kernels_b200.npz, produced by tests/golden/make_ref_golden.py).

This is what pins the oracle: copies and conv arithmetic must match bit for bit,
K/q after RMSNorm+RoPE within one f16 ulp (the GPU's rsqrt.approx is not correctly
rounded), attention within the 2e-3 bar (the oracle's exp2 is correctly rounded, the
GPU's ex2.approx is not)."""
import importlib.util
import os

import numpy as np
import pytest

from oracle import cpu as O
from tests.kvcase import DecodeCase, ulp_diff_f16

HERE = os.path.dirname(os.path.abspath(__file__))
spec = importlib.util.spec_from_file_location("make_ref_golden", os.path.join(HERE, "golden", "make_ref_golden.py"))
G = importlib.util.module_from_spec(spec)
spec.loader.exec_module(G)


@pytest.fixture(scope="module")
def gold():
    return np.load(os.path.join(HERE, "golden", "ref_kernels_b200.npz"))


def _bits(a):
    return np.ascontiguousarray(a).view(np.uint16)


def _append(case):
    h = case.host()
    O.qk_rmsnorm(h.q, case.q_norm_w)
    O.qk_rmsnorm(h.k, case.k_norm_w)
    O.rope(h.q, case.cos, case.sin, case.pos_ids)
    O.rope(h.k, case.cos, case.sin, case.pos_ids)
    O.kv_copy(h.k_ptrs, h.k, case.pos_ids)
    O.kv_copy(h.v_ptrs, h.v, case.pos_ids)
    return h


def test_append_matches_reference_kernels(gold):
    case = DecodeCase(G.DECODE_LENS, seed=G.DECODE_SEED)
    h = _append(case)
    v_rows = np.stack([h.v_cache[i][int(n)] for i, n in enumerate(case.lens)])
    k_rows = np.stack([h.k_cache[i][int(n)] for i, n in enumerate(case.lens)])
    assert np.array_equal(_bits(v_rows), _bits(gold["v_rows"]))           # byte copy
    assert ulp_diff_f16(k_rows, gold["k_rows"]).max() <= 1
    dq = ulp_diff_f16(h.q, gold["q_after_append"])
    assert dq.max() <= 1 and (dq != 0).mean() < 0.02


@pytest.mark.parametrize("window", G.WINDOWS)
def test_decode_attention_matches_reference_kernels(gold, window):
    case = DecodeCase(G.DECODE_LENS, seed=G.DECODE_SEED)
    h = _append(case)
    # feed the reference's own q (removes the 1-ulp q differences from the comparison)
    q = np.ascontiguousarray(gold["q_after_append"])
    for i, n in enumerate(case.lens):
        h.k_cache[i][int(n)] = gold["k_rows"][i]
    online = O.attn_online(q, h.k_ptrs, h.v_ptrs, case.seq_lens, window)
    assert np.abs(online.astype(np.float32) - gold[f"ctx_online_ungated_w{window}"].astype(np.float32)).max() <= 1e-3
    acc, stats = O.attn_split(q, h.k_ptrs, h.v_ptrs, case.seq_lens, window)
    gs = gold[f"partial_stats_w{window}"]
    assert stats.shape == gs.shape
    live = gs[..., 1] > 0  # key ranges that hold keys
    assert np.allclose(stats[..., 0][live], gs[..., 0][live], rtol=0, atol=2e-5)      # running max
    assert np.allclose(stats[..., 1][live], gs[..., 1][live], rtol=2e-5, atol=1e-6)   # normaliser
    ctx = O.attn_combine(acc, stats)
    O.sigmoid_gate(ctx, case.gate)
    assert np.abs(ctx.astype(np.float32) - gold[f"ctx_gated_w{window}"].astype(np.float32)).max() <= 1e-3


def test_conv_decode_matches_reference_kernel_bitwise(gold):
    state, bcx, w = G.conv_inputs()
    y = O.conv_decode(O.ptr_table(state), bcx, w)
    assert np.array_equal(_bits(y), _bits(gold["conv_y"]))
    assert np.array_equal(_bits(np.stack(state)), _bits(gold["conv_state"]))


def test_conv_state_prefill_matches_reference_kernel_bitwise(gold):
    bcx, carry, origin, lpos, owner = G.conv_prefill_inputs()
    pool = O.conv_state_prefill(O.ptr_table([carry[i] for i in owner]), origin, lpos, bcx)
    assert np.array_equal(_bits(pool), _bits(gold["conv_pool"]))
