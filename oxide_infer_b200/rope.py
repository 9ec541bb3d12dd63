"""Host-side RoPE table generator with the reference's table format
(crates/oxide-infer-models/src/rope.rs:158-201): f16 cos/sin [max_pos][128],
inv_freq[i] = 1/theta^(2i/128) for i < floor(partial*128)/2 else 0, the 64
angles repeated for dims 64..127, all arithmetic in float32."""
from __future__ import annotations

import numpy as np


def rotary_tables(max_seq_len: int, rope_theta: float = 1e6, partial_rotary_factor: float = 0.5,
                  head_dim: int = 128):
    half = head_dim // 2
    angles = int(np.float32(partial_rotary_factor) * np.float32(head_dim)) // 2
    inv = np.zeros(half, np.float32)
    i = np.arange(min(angles, half), dtype=np.float32)
    inv[: len(i)] = np.float32(1.0) / np.power(np.float32(rope_theta),
                                               (np.float32(2.0) * i) / np.float32(head_dim),
                                               dtype=np.float32)
    pos = np.arange(max_seq_len, dtype=np.float32)[:, None]
    ang = (pos * np.concatenate([inv, inv])[None, :]).astype(np.float32)
    return np.cos(ang, dtype=np.float32).astype(np.float16), np.sin(ang, dtype=np.float32).astype(np.float16)
