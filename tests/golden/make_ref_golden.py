"""Generates tests/golden/ref_kernels_b200.npz by running the REFERENCE's own kernels
(oracle/_ref/*.cubin, built from the reference's PTX by oracle/build_ref.py) on a B200.

    python tests/golden/make_ref_golden.py        # needs a CUDA device and oracle/_ref/

The fixture holds only outputs; the inputs are regenerated from the seeds below by
tests/kvcase.DecodeCase and the helper functions in this file, which the CPU test
(tests/test_golden_ref.py) imports.  Keep the cases small: the file is committed."""
from __future__ import annotations

import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_kernels_b200.npz")
HIDDEN = 2048

DECODE_LENS = [63, 64, 130, 300]   # old lengths; the appended token makes 64, 65, 131, 301 keys
DECODE_SEED = 11
WINDOWS = [0, 256]
CONV_SEED, CONV_B = 12, 2
PREFILL_LENS = [1, 5, 9]           # conv prefill chunks
PREFILL_SEED = 13


def conv_inputs():
    rng = np.random.default_rng(CONV_SEED)
    state = [rng.standard_normal((HIDDEN, 6), dtype=np.float32).astype(np.float16) for _ in range(CONV_B)]
    bcx = rng.standard_normal((CONV_B, 3 * HIDDEN), dtype=np.float32).astype(np.float16)
    w = (rng.standard_normal((HIDDEN, 7), dtype=np.float32) * 0.1).astype(np.float16)
    return state, bcx, w


def conv_prefill_inputs():
    rng = np.random.default_rng(PREFILL_SEED)
    rows = sum(PREFILL_LENS)
    bcx = rng.standard_normal((rows, 3 * HIDDEN), dtype=np.float32).astype(np.float16)
    carry = [rng.standard_normal((HIDDEN, 6), dtype=np.float32).astype(np.float16) for _ in PREFILL_LENS]
    origin, lpos, owner = [], [], []
    r0 = 0
    for i, n in enumerate(PREFILL_LENS):
        origin += [r0] * n
        lpos += list(range(n))
        owner += [i] * n
        r0 += n
    return bcx, carry, np.array(origin, np.uint32), np.array(lpos, np.uint32), owner


def main():
    import torch
    from oracle.refptx import RefPtx
    from tests.kvcase import DecodeCase, dev_ptr_table, u32
    ref = RefPtx()
    out = {}
    case = DecodeCase(DECODE_LENS, seed=DECODE_SEED)
    b = case.b
    for window in WINDOWS:
        d = case.device()
        ref.append(d.q, d.k, d.v, d.q_norm_w, d.k_norm_w, d.cos, d.sin, d.pos_ids, d.k_ptrs, d.v_ptrs, b)
        nch = ref.nchunks_for(int(case.seq_lens.max()), window)
        acc = torch.zeros(b * nch * 16 * 128, dtype=torch.float32, device="cuda")
        stats = torch.zeros(b * nch * 16 * 2, dtype=torch.float32, device="cuda")
        ref.decode_attention(d.ctx, d.q, d.gate, d.k_ptrs, d.v_ptrs, d.seq_lens, b, window,
                             int(case.seq_lens.max()), acc, stats)
        online = torch.zeros_like(d.ctx)
        ref.attn_online(online, d.q, d.k_ptrs, d.v_ptrs, d.seq_lens, b, window)
        torch.cuda.synchronize()
        if window == 0:
            out["q_after_append"] = d.q.cpu().numpy()
            out["k_rows"] = np.stack([d.k_cache[i][int(n)].cpu().numpy() for i, n in enumerate(case.lens)])
            out["v_rows"] = np.stack([d.v_cache[i][int(n)].cpu().numpy() for i, n in enumerate(case.lens)])
        out[f"ctx_gated_w{window}"] = d.ctx.cpu().numpy()
        out[f"ctx_online_ungated_w{window}"] = online.cpu().numpy()
        out[f"partial_stats_w{window}"] = stats.cpu().numpy().reshape(b, nch, 16, 2)
    # conv decode
    state, bcx, w = conv_inputs()
    ds = [torch.from_numpy(s.copy()).cuda() for s in state]
    y = torch.zeros(CONV_B, HIDDEN, dtype=torch.float16, device="cuda")
    ref.conv_decode(y, dev_ptr_table(ds), torch.from_numpy(bcx).cuda(), torch.from_numpy(w).cuda(), CONV_B)
    torch.cuda.synchronize()
    out["conv_y"] = y.cpu().numpy()
    out["conv_state"] = np.stack([s.cpu().numpy() for s in ds])
    # conv prefill: gathered pool rows
    pbcx, carry, origin, lpos, owner = conv_prefill_inputs()
    rows = pbcx.shape[0]
    dc = [torch.from_numpy(c.copy()).cuda() for c in carry]
    pool = torch.zeros(rows, HIDDEN, 6, dtype=torch.float16, device="cuda")
    ref.conv_state_prefill(pool, dev_ptr_table([dc[i] for i in owner]), u32(origin), u32(lpos),
                           torch.from_numpy(pbcx).cuda(), rows)
    torch.cuda.synchronize()
    out["conv_pool"] = pool.cpu().numpy()
    np.savez_compressed(OUT, **out)
    print("wrote", OUT, os.path.getsize(OUT), "bytes")


if __name__ == "__main__":
    main()
