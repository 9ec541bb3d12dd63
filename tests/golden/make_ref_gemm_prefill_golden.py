"""Generates tests/golden/ref_gemm_prefill_b200.npz: outputs of the REFERENCE's GEMM prefill kernels
(batched_attn_pack_q_fp16, batched_attn_softmax_mask_fp16, batched_attn_gate_scatter_fp16,
batched_attn.rs:2283-2645; cubins in oracle/_ref/ built from the reference's PTX by
oracle/build_ref.py) run on a B200 in the engine's order (batch_engine.rs:439-592), with a torch
float32 matmul on the same f16 operands standing in for each of the two cuBLASLt calls between them.

    python tests/golden/make_ref_gemm_prefill_golden.py [out.npz]    # needs a CUDA device and oracle/_ref/

Cases: the reference's own chunk shapes (test_gemm_attention.rs: 96 rows at position 0, 128 rows at
position 400) with windows 0 and 256.  The fixture holds outputs only (the softmax column sums in full,
the context of KEEP_ROWS rows per case); the inputs are regenerated from the seeds by chunk_inputs(),
which the tests import."""
from __future__ import annotations

import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_gemm_prefill_b200.npz")
NQ, NKV, HD = 16, 4, 128
CASES = [(96, 0, 0), (96, 0, 256), (128, 400, 0), (128, 400, 256)]   # (rows, first position, window)
SEED = 21


def chunk_inputs(rows, p0, seed=SEED):
    rng = np.random.default_rng(seed + rows + p0)
    f16 = lambda *s: rng.standard_normal(s, dtype=np.float32).astype(np.float16)
    return {"q": f16(rows, NQ, HD), "gate": f16(rows, NQ), "k": f16(p0 + rows, NKV, HD), "v": f16(p0 + rows, NKV, HD)}


def keep_rows(rows):
    """Rows whose context is stored: the first and last eight and eight spread between."""
    mid = np.linspace(8, rows - 9, 8).astype(int)
    return sorted(set(range(8)) | set(range(rows - 8, rows)) | set(int(m) for m in mid))


def case_name(rows, p0, window):
    return f"r{rows}_p{p0}_w{window}"


def main():
    import torch
    from oracle.refptx import RefPtx
    ref = RefPtx()
    out = {}
    for rows, p0, window in CASES:
        x = chunk_inputs(rows, p0)
        d = {k: torch.from_numpy(v).cuda() for k, v in x.items()}
        seq_lens = torch.arange(p0 + 1, p0 + rows + 1, dtype=torch.int32, device="cuda")
        ctx = torch.zeros(rows, NQ, HD, dtype=torch.float16, device="cuda")
        sums = ref.gemm_attention_chunk(ctx, d["q"], d["gate"], d["k"], d["v"], seq_lens, rows, p0 + 1, p0 + rows, window)
        torch.cuda.synchronize()
        name = case_name(rows, p0, window)
        out["ctx_" + name] = ctx.cpu().numpy()[keep_rows(rows)]
        out["sums_" + name] = sums.cpu().numpy()
    path = sys.argv[1] if len(sys.argv) > 1 else OUT
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
