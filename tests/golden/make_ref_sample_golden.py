"""Generates tests/golden/ref_sample_b200.npz by running the REFERENCE's own argmax and
embedding-lookup kernels (oracle/_ref/*.cubin, built from the reference's PTX by
oracle/build_ref.py) on a B200.

    python tests/golden/make_ref_sample_golden.py [--out FILE]    # needs a CUDA device and oracle/_ref/

The fixture holds only outputs (token ids, gathered rows); the inputs are regenerated from the
seeds below by sample_cases() / embed_case(), which the tests import."""
from __future__ import annotations

import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_sample_b200.npz")
VOCAB = 128000  # batch_engine.rs:75


def sample_cases():
    """name -> logits [batch][vocab] f16.  Ties, NaN and infinities are there on purpose: the
    reference resolves equal maxima by its scan order and reduction tree."""
    rng = np.random.default_rng(21)
    cases = {}
    cases["normal_4x128000"] = rng.standard_normal((4, VOCAB), dtype=np.float32).astype(np.float16)
    # few distinct values: hundreds of equal maxima per row
    cases["quantised_8x128000"] = (np.round(rng.standard_normal((8, VOCAB), dtype=np.float32) * 1.5) / 2).astype(np.float16)
    cases["clipped_3x1001"] = np.minimum(rng.standard_normal((3, 1001), dtype=np.float32), 0.75).astype(np.float16)
    cases["short_2x100"] = np.minimum(rng.standard_normal((2, 100), dtype=np.float32), 0.5).astype(np.float16)
    cases["zeros_1x5000"] = np.zeros((1, 5000), np.float16)
    last = rng.standard_normal((2, 4096), dtype=np.float32).astype(np.float16)
    last[0, 4095] = 9.0
    last[1, 0] = 9.0
    cases["ends_2x4096"] = last
    sp = rng.standard_normal((4, 3000), dtype=np.float32).astype(np.float16)
    sp[0, ::7] = np.nan
    sp[0, [100, 2000]] = np.inf
    sp[1, :] = -np.inf
    sp[2, :] = np.nan
    sp[3, 17] = np.inf
    sp[3, 1041] = np.inf  # same virtual thread (17 + 4*256): the first one stays
    cases["special_4x3000"] = sp
    return cases


def embed_case():
    rng = np.random.default_rng(22)
    table = rng.standard_normal((512, 2048), dtype=np.float32).astype(np.float16)
    ids = np.array([0, 511, 7, 7, 300, 1, 255, 256], np.uint32)
    return table, ids


def main():
    import torch
    from oracle.refptx import RefPtx
    out_path = OUT
    if "--out" in sys.argv:
        out_path = sys.argv[sys.argv.index("--out") + 1]
    ref = RefPtx()
    out = {}
    for name, logits in sample_cases().items():
        d = torch.from_numpy(logits).cuda()
        tok = torch.zeros(logits.shape[0], dtype=torch.int32, device="cuda")
        ref.argmax(tok, d, logits.shape[1], logits.shape[0])
        torch.cuda.synchronize()
        out["argmax_" + name] = tok.cpu().numpy().astype(np.uint32)
    table, ids = embed_case()
    dt, di = torch.from_numpy(table).cuda(), torch.from_numpy(ids.astype(np.int32)).cuda()
    o = torch.zeros(ids.shape[0], table.shape[1], dtype=torch.float16, device="cuda")
    ref.embed_lookup(o, dt, di, table.shape[1], ids.shape[0])
    torch.cuda.synchronize()
    out["embed_rows"] = o.cpu().numpy()
    np.savez_compressed(out_path, **out)
    print("wrote", out_path, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
