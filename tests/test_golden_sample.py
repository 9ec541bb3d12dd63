"""The CPU oracle's argmax / embedding lookup against outputs of the REFERENCE's own kernels run
on a B200 (tests/golden/ref_sample_b200.npz, produced by tests/golden/make_ref_sample_golden.py),
plus hand-derived known answers for the tie rule."""
import importlib.util
import os

import numpy as np

from oracle import cpu as O

HERE = os.path.dirname(os.path.abspath(__file__))
spec = importlib.util.spec_from_file_location("make_ref_sample_golden", os.path.join(HERE, "golden", "make_ref_sample_golden.py"))
G = importlib.util.module_from_spec(spec)
spec.loader.exec_module(G)


def test_oracle_argmax_matches_reference_kernel_outputs():
    gold = np.load(os.path.join(HERE, "golden", "ref_sample_b200.npz"))
    for name, logits in G.sample_cases().items():
        assert np.array_equal(O.argmax(logits), gold["argmax_" + name]), name


def test_oracle_embed_matches_reference_kernel_outputs():
    gold = np.load(os.path.join(HERE, "golden", "ref_sample_b200.npz"))
    table, ids = G.embed_case()
    assert np.array_equal(O.embed_lookup(table, ids).view(np.uint16), gold["embed_rows"].view(np.uint16))


def test_argmax_known_answers():
    # no ties: plain argmax
    rng = np.random.default_rng(1)
    x = rng.permutation(5000).astype(np.float32).reshape(2, 2500)
    x = (x / 4).astype(np.float16)  # distinct values stay distinct (multiples of 0.25 below 2048)
    assert np.array_equal(O.argmax(x), x.astype(np.float32).argmax(1))
    # equal maxima at 8 and 16 (lanes 8 and 16 of warp 0): offset 16 moves lane 16's pair to lane 0,
    # offset 8 then compares it with lane 8's equal value and keeps it -> 16, not the lowest index
    y = np.zeros((1, 1000), np.float16)
    y[0, [8, 16]] = 1
    assert O.argmax(y)[0] == 16
    # equal maxima in one thread's stripe (3 and 3 + 256): the first one stays
    y = np.zeros((1, 1000), np.float16)
    y[0, [3, 259]] = 1
    assert O.argmax(y)[0] == 3
    # equal maxima in warps 2 and 4 (indices 64 and 128): at offset 4 warp 0's slot takes warp 4's pair
    # (strictly greater than its own 0), at offset 2 it meets warp 2's equal value and keeps its own
    y = np.zeros((1, 1000), np.float16)
    y[0, [64, 128]] = 1
    assert O.argmax(y)[0] == 128
    # equal maxima in warps 0 and 4: warp 0's own pair is never replaced by an equal one
    y = np.zeros((1, 1000), np.float16)
    y[0, [0, 128]] = 1
    assert O.argmax(y)[0] == 0
    # nothing above -1e30 / only NaN: index 0
    assert O.argmax(np.full((1, 300), -np.inf, np.float16))[0] == 0
    assert O.argmax(np.full((1, 300), np.nan, np.float16))[0] == 0
