"""ctypes front end of the CPU oracle (TEST INFRASTRUCTURE ONLY).

Only tests, ``__graft_entry__.smoke()`` and the CPU-baseline leg of
``bench.py`` may import this module.  The product package never does.

All f16 tensors are ``numpy.float16`` arrays (C-contiguous); pointer tables are
``numpy.uint64`` arrays holding host addresses of such arrays.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "liboxi_oracle.so")

NQ, NKV, HD, KV_DIM, HIDDEN, CONV_K = 16, 4, 128, 512, 2048, 7
ATTN_SCALE = 0.0883883476


def build(force: bool = False) -> str:
    """Compile liboxi_oracle.so next to its source if it is missing or stale."""
    src = os.path.join(_HERE, "oxi_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B"], check=True, capture_output=True)
    return _SO


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_SO)
        L.orc_pat.restype = C.c_float
        L.orc_pat.argtypes = [C.c_uint64, C.c_uint64]
        L.orc_h2f.restype = C.c_float
        L.orc_h2f.argtypes = [C.c_uint16]
        L.orc_f2h.restype = C.c_uint16
        L.orc_f2h.argtypes = [C.c_float]
        L.orc_num_threads.restype = C.c_int
        L.orc_set_num_threads.restype = None
        L.orc_set_num_threads.argtypes = [C.c_int]
        _lib = L
    return _lib


def _p(a: np.ndarray | None):
    if a is None:
        return C.c_void_p(0)
    assert a.flags["C_CONTIGUOUS"], "oracle arrays must be contiguous"
    return C.c_void_p(a.ctypes.data)


def _u32(v):
    return C.c_uint32(int(v))


def num_threads() -> int:
    return int(lib().orc_num_threads())


def use_all_cores() -> int:
    """Lets the OpenMP loops use every core this process may run on, whatever OMP_NUM_THREADS says
    (torch.distributed.run exports OMP_NUM_THREADS=1 to its workers).  Returns the thread count."""
    import os
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    lib().orc_set_num_threads(n)
    return num_threads()


# --------------------------------------------------------------- helpers --

def pat(seed: int, n: int, scale: float = 1.0) -> np.ndarray:
    """``pat(seed, i) * scale`` for i in [0, n) as float32 (reference generator)."""
    out = np.empty(n, np.float32)
    lib().orc_pat_fill(C.c_uint64(seed), C.c_float(scale), _p(out), C.c_size_t(n))
    return out


def pat_numpy(seed: int, n: int) -> np.ndarray:
    """Independent numpy statement of the same generator (for cross-checking)."""
    with np.errstate(over="ignore"):
        x = np.uint64(seed) * np.uint64(6364136223846793005) + np.arange(n, dtype=np.uint64)
        x ^= x >> np.uint64(33)
        x *= np.uint64(0xFF51AFD7ED558CCD)
        x ^= x >> np.uint64(33)
    return ((x & np.uint64(0xFFFF)).astype(np.float32) / np.float32(32767.5)) - np.float32(1.0)


def f2h(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32)
    out = np.empty(x.shape, np.uint16)
    lib().orc_f2h_array(_p(x), _p(out), C.c_size_t(x.size))
    return out.view(np.float16)


def rope_table(max_pos: int, theta: float = 1e6, partial: float = 0.5, hd: int = HD):
    cos = np.empty((max_pos, hd), np.float16)
    sin = np.empty((max_pos, hd), np.float16)
    lib().orc_rope_table(_p(cos), _p(sin), _u32(max_pos), _u32(hd), C.c_float(theta),
                         C.c_float(partial))
    return cos, sin


def ptr_table(arrays) -> np.ndarray:
    """uint64 table of host addresses, one per array (the k_ptrs/v_ptrs/conv_ptrs analogue)."""
    return np.array([a.ctypes.data for a in arrays], np.uint64)


# ------------------------------------------------------------- operators --

def qk_rmsnorm(x_io, w, eps=1e-5):
    b, heads, hd = x_io.shape
    lib().orc_qk_rmsnorm(_p(x_io), _p(w), C.c_float(eps), _u32(heads), _u32(hd), _u32(b))


def rope(x_io, cos, sin, pos_ids):
    b, heads, hd = x_io.shape
    lib().orc_rope(_p(x_io), _p(cos), _p(sin), _p(pos_ids), _u32(heads), _u32(hd), _u32(b))


def kv_copy(dst_ptrs, src, pos_ids):
    b = src.shape[0]
    lib().orc_kv_copy(_p(dst_ptrs), _p(src), _p(pos_ids), _u32(src.size // b), _u32(b))


def attn_online(q, k_ptrs, v_ptrs, seq_lens, window=0):
    b = q.shape[0]
    ctx = np.empty((b, NQ, HD), np.float16)
    lib().orc_attn_online(_p(ctx), _p(q), _p(k_ptrs), _p(v_ptrs), _p(seq_lens), _u32(b), _u32(window))
    return ctx


def attn_split(q, k_ptrs, v_ptrs, seq_lens, window=0, chunk_keys=128, nchunks=None):
    b = q.shape[0]
    if nchunks is None:
        eff = [int(s) if window == 0 else min(int(s), window) for s in seq_lens]
        nchunks = max(1, max(-(-e // chunk_keys) for e in eff))
    acc = np.zeros((b, nchunks, NQ, HD), np.float32)
    stats = np.zeros((b, nchunks, NQ, 2), np.float32)
    lib().orc_attn_split(_p(q), _p(k_ptrs), _p(v_ptrs), _p(seq_lens), _p(acc), _p(stats), _u32(b),
                         _u32(window), _u32(chunk_keys), _u32(nchunks))
    return acc, stats


def attn_combine(acc, stats):
    b, nchunks = acc.shape[:2]
    ctx = np.empty((b, NQ, HD), np.float16)
    lib().orc_attn_combine(_p(ctx), _p(acc), _p(stats), _u32(b), _u32(nchunks))
    return ctx


def sigmoid_gate(ctx_io, gate):
    b, heads, hd = ctx_io.shape
    lib().orc_sigmoid_gate(_p(ctx_io), _p(gate), _u32(heads), _u32(hd), _u32(b))


def decode_attn(q, gate, k_ptrs, v_ptrs, seq_lens, window=0):
    """split4+combine (or online when one chunk) then the gate: BE:1155-1239."""
    eff = [int(s) if window == 0 else min(int(s), window) for s in seq_lens]
    nchunks = max(1, max(-(-e // 128) for e in eff))
    if nchunks > 1:
        ctx = attn_combine(*attn_split(q, k_ptrs, v_ptrs, seq_lens, window, 128, nchunks))
    else:
        ctx = attn_online(q, k_ptrs, v_ptrs, seq_lens, window)
    if gate is not None:
        sigmoid_gate(ctx, gate)
    return ctx


def decode_layer(q_io, k_io, v_in, gate, q_norm_w, k_norm_w, cos, sin, pos_ids, seq_lens,
                 k_ptrs, v_ptrs, window=0, eps=1e-5):
    """Whole attention-layer decode sequence (in place on q_io/k_io and the caches)."""
    b = q_io.shape[0]
    eff = [int(s) if window == 0 else min(int(s), window) for s in seq_lens]
    nchunks = max(1, max(-(-e // 128) for e in eff))
    ctx = np.empty((b, NQ, HD), np.float16)
    acc = np.empty((b, nchunks, NQ, HD), np.float32)
    stats = np.empty((b, nchunks, NQ, 2), np.float32)
    lib().orc_decode_layer(_p(ctx), _p(q_io), _p(k_io), _p(v_in), _p(gate), _p(q_norm_w),
                           _p(k_norm_w), _p(cos), _p(sin), _p(pos_ids), _p(seq_lens), _p(k_ptrs),
                           _p(v_ptrs), _u32(b), _u32(window), C.c_float(eps), _p(acc), _p(stats),
                           _u32(nchunks))
    return ctx


def linear(x, w):
    """y = f16(x @ w.T) with f32 accumulation in index order (the projection GEMMs, lt.gemm)."""
    rows, out = x.shape[0], w.shape[0]
    y = np.empty((rows, out), np.float16)
    lib().orc_linear_f16(_p(y), _p(x), _p(w), _u32(rows), _u32(out), _u32(x.shape[1]))
    return y


def prefill_gemm_chunk(q, gate, k_cache, v_cache, p0, window=0):
    rows = q.shape[0]
    ctx = np.empty((rows, NQ, HD), np.float16)
    lib().orc_prefill_gemm_chunk(_p(ctx), _p(q), _p(gate), _p(k_cache), _p(v_cache), _u32(rows),
                                 _u32(p0), _u32(window))
    return ctx


def conv_decode(state_ptrs, bcx, conv_w):
    b = bcx.shape[0]
    hidden = bcx.shape[1] // 3
    y = np.empty((b, hidden), np.float16)
    lib().orc_conv_decode(_p(y), _p(state_ptrs), _p(bcx), _p(conv_w), _u32(hidden),
                          _u32(conv_w.shape[1]), _u32(b))
    return y


def conv_state_prefill(carry_tbl, origin, local_pos, bcx, k_len=CONV_K):
    rows = bcx.shape[0]
    hidden = bcx.shape[1] // 3
    pool = np.empty((rows, hidden, 6), np.float16)
    lib().orc_conv_state_prefill(_p(pool), _p(carry_tbl), _p(origin), _p(local_pos), _p(bcx),
                                 _u32(hidden), _u32(k_len), _u32(rows))
    return pool


def conv_prefill_wave(carry_tbl, origin, local_pos, bcx, conv_w):
    """Gather + conv on every row + copy-back of each chunk's final state (in place)."""
    rows = bcx.shape[0]
    hidden = bcx.shape[1] // 3
    y = np.empty((rows, hidden), np.float16)
    pool = np.empty((rows, hidden, 6), np.float16)
    lib().orc_conv_prefill_wave(_p(y), _p(pool), _p(carry_tbl), _p(origin), _p(local_pos), _p(bcx),
                                _p(conv_w), _u32(hidden), _u32(conv_w.shape[1]), _u32(rows))
    return y


def embed_lookup(table, token_ids):
    """out[b] = table[token_ids[b]] (batched_embed_lookup_fp16)."""
    table = np.ascontiguousarray(table, np.float16)
    tok = np.ascontiguousarray(token_ids, np.uint32)
    out = np.empty((tok.shape[0], table.shape[1]), np.float16)
    lib().orc_embed_lookup(_p(out), _p(table), _p(tok), _u32(table.shape[1]), _u32(tok.shape[0]))
    return out


def argmax(logits, nthreads=256):
    """Per-row argmax with the reference kernel's scan order and reduction tree (batched_argmax_direct_f16)."""
    logits = np.ascontiguousarray(logits, np.float16)
    out = np.empty(logits.shape[0], np.uint32)
    lib().orc_argmax(_p(out), _p(logits), _u32(logits.shape[1]), _u32(logits.shape[0]), _u32(nthreads))
    return out


# ------------------------------------------------ f64 mathematical model --

def attention_f64(q, k_cache, v_cache, slen, window=0, gate=None):
    """Exact softmax attention in float64 for one row (the form of the host
    references in test_split_attention.rs:41-72 and test_gemm_attention.rs:59-104).
    q [16][128], caches [>=slen][4][128]; any float dtype.  Returns float64 [16][128]."""
    q = np.asarray(q, np.float64).reshape(NQ, HD)
    k = np.asarray(k_cache, np.float64).reshape(-1, NKV, HD)[:slen]
    v = np.asarray(v_cache, np.float64).reshape(-1, NKV, HD)[:slen]
    t0 = slen - window if (window and slen > window) else 0
    out = np.empty((NQ, HD))
    for h in range(NQ):
        kv = h // 4
        s = (k[t0:, kv] @ q[h]) * ATTN_SCALE
        w = np.exp(s - s.max())
        out[h] = (w[:, None] * v[t0:, kv]).sum(0) / w.sum()
        if gate is not None:
            out[h] *= 1.0 / (1.0 + np.exp(-float(np.asarray(gate).reshape(-1)[h])))
    return out
