"""Seeded synthetic cases shared by the GPU parity tests, smoke() and bench.py.

A case holds the same data twice: numpy arrays addressed by host pointer tables
(for the CPU oracle) and torch CUDA tensors addressed by device pointer tables
(for the library and for the reference's kernels)."""
from __future__ import annotations

import numpy as np
import torch

NQ, NKV, HD, HIDDEN = 16, 4, 128, 2048


# ---- guard bands: out-of-bounds evidence without a sanitizer -------------------------------
# Every buffer a kernel may write through a table (K/V caches, conv states, contexts) can be
# placed between two bands of a fixed byte pattern inside one allocation.  A write that lands
# before or behind the buffer changes a band; check_guards() (run after every GPU test by
# tests/conftest.py) finds it.  Without the bands such a write would land in a neighbouring torch
# allocation and pass unnoticed.
GUARD_BYTES = 4096
GUARD_BYTE = 0xA5
_GUARDS = []  # (whole allocation as uint8, payload bytes, label)


def guarded(a, label="buffer"):
    """Copies numpy array (or CPU tensor) `a` to the GPU between two guard bands; returns the
    payload view (same shape and dtype, 16-byte aligned)."""
    t = torch.from_numpy(np.ascontiguousarray(a)) if isinstance(a, np.ndarray) else a.contiguous()
    nbytes = t.numel() * t.element_size()
    pad = (-nbytes) % 16
    whole = torch.full((GUARD_BYTES + nbytes + pad + GUARD_BYTES,), GUARD_BYTE, dtype=torch.uint8, device="cuda")
    payload = whole[GUARD_BYTES:GUARD_BYTES + nbytes].view(t.dtype).view(t.shape)
    payload.copy_(t)
    _GUARDS.append((whole, nbytes, label))
    return payload


def check_guards(clear=True):
    """Asserts that no guard band registered since the last call was written to; returns how many
    buffers were checked."""
    n = len(_GUARDS)
    bad = []
    for whole, nbytes, label in _GUARDS:
        front = whole[:GUARD_BYTES]
        back = whole[GUARD_BYTES + nbytes:]
        if not (bool((front == GUARD_BYTE).all()) and bool((back == GUARD_BYTE).all())):
            bad.append(label)
    if clear:
        _GUARDS.clear()
    assert not bad, f"out-of-bounds write next to: {bad[:8]} ({len(bad)} of {n} guarded buffers)"
    return n


def u32(t):  # numpy uint32 -> torch int32 bit pattern on the GPU
    return torch.from_numpy(np.ascontiguousarray(t).view(np.int32)).cuda()


def dev_ptr_table(tensors):
    return torch.tensor([t.data_ptr() for t in tensors], dtype=torch.int64, device="cuda")


class DecodeCase:
    """One attention layer, one decode step: `lens` old tokens per sequence, one appended."""

    def __init__(self, lens, seed=0, theta=1e6, partial=0.5, max_pos=None, spare_rows=1,
                 kscale=1.0):
        from oracle import cpu as O
        rng = np.random.default_rng(seed)
        self.lens = np.asarray(lens, np.uint32)
        b = self.b = len(self.lens)
        f16 = lambda *s, sc=1.0: (rng.standard_normal(s, dtype=np.float32) * sc).astype(np.float16)
        self.k_cache = [f16(int(n) + spare_rows, NKV, HD, sc=kscale) for n in self.lens]
        self.v_cache = [f16(int(n) + spare_rows, NKV, HD) for n in self.lens]
        self.q, self.k, self.v = f16(b, NQ, HD), f16(b, NKV, HD), f16(b, NKV, HD)
        self.gate = f16(b, NQ)
        self.q_norm_w = (1 + 0.02 * rng.standard_normal(HD)).astype(np.float16)
        self.k_norm_w = (1 + 0.02 * rng.standard_normal(HD)).astype(np.float16)
        mp = int(max_pos or (int(self.lens.max()) + 2))
        self.cos, self.sin = O.rope_table(mp, theta, partial)
        self.pos_ids = self.lens.copy()
        self.seq_lens = self.lens + 1

    # ---- host (oracle) view: fresh copies so the case can be replayed
    def host(self):
        from oracle import cpu as O
        h = type("H", (), {})()
        h.k_cache = [a.copy() for a in self.k_cache]
        h.v_cache = [a.copy() for a in self.v_cache]
        h.k_ptrs, h.v_ptrs = O.ptr_table(h.k_cache), O.ptr_table(h.v_cache)
        h.q, h.k, h.v = self.q.copy(), self.k.copy(), self.v.copy()
        return h

    # ---- device view
    def device(self):
        d = type("D", (), {})()
        d.k_cache = [guarded(a, f"k_cache[{i}]") for i, a in enumerate(self.k_cache)]
        d.v_cache = [guarded(a, f"v_cache[{i}]") for i, a in enumerate(self.v_cache)]
        d.k_ptrs, d.v_ptrs = dev_ptr_table(d.k_cache), dev_ptr_table(d.v_cache)
        d.q, d.k, d.v = (torch.from_numpy(x.copy()).cuda() for x in (self.q, self.k, self.v))
        d.gate = torch.from_numpy(self.gate).cuda()
        d.q_norm_w = torch.from_numpy(self.q_norm_w).cuda()
        d.k_norm_w = torch.from_numpy(self.k_norm_w).cuda()
        d.cos, d.sin = torch.from_numpy(self.cos).cuda(), torch.from_numpy(self.sin).cuda()
        d.pos_ids, d.seq_lens = u32(self.pos_ids), u32(self.seq_lens)
        d.ctx = guarded(np.zeros((self.b, NQ, HD), np.float16), "ctx")
        return d


def ulp_diff_f16(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """Distance in f16 representable steps between two float16 arrays (finite values)."""
    def key(x):
        u = x.view(np.uint16).astype(np.int32)
        return np.where(u & 0x8000, 0x8000 - u, u)  # monotone integer order
    return np.abs(key(a) - key(b))
