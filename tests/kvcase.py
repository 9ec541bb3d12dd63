"""Seeded synthetic cases shared by the GPU parity tests, smoke() and bench.py.

A case holds the same data twice: numpy arrays addressed by host pointer tables
(for the CPU oracle) and torch CUDA tensors addressed by device pointer tables
(for the library and for the reference's kernels)."""
from __future__ import annotations

import numpy as np
import torch

NQ, NKV, HD, HIDDEN = 16, 4, 128, 2048


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
        d.k_cache = [torch.from_numpy(a).cuda() for a in self.k_cache]
        d.v_cache = [torch.from_numpy(a).cuda() for a in self.v_cache]
        d.k_ptrs, d.v_ptrs = dev_ptr_table(d.k_cache), dev_ptr_table(d.v_cache)
        d.q, d.k, d.v = (torch.from_numpy(x.copy()).cuda() for x in (self.q, self.k, self.v))
        d.gate = torch.from_numpy(self.gate).cuda()
        d.q_norm_w = torch.from_numpy(self.q_norm_w).cuda()
        d.k_norm_w = torch.from_numpy(self.k_norm_w).cuda()
        d.cos, d.sin = torch.from_numpy(self.cos).cuda(), torch.from_numpy(self.sin).cuda()
        d.pos_ids, d.seq_lens = u32(self.pos_ids), u32(self.seq_lens)
        d.ctx = torch.zeros(self.b, NQ, HD, dtype=torch.float16, device="cuda")
        return d


def ulp_diff_f16(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """Distance in f16 representable steps between two float16 arrays (finite values)."""
    def key(x):
        u = x.view(np.uint16).astype(np.int32)
        return np.where(u & 0x8000, 0x8000 - u, u)  # monotone integer order
    return np.abs(key(a) - key(b))
