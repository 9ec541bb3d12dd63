"""Runs the reference's own kernels (cubins in oracle/_ref/) on the GPU.

TEST INFRASTRUCTURE ONLY: used by the ``-m gpu`` parity tests, the fixture
generator under tests/golden/ and the reference arm of ``bench.py``.  Grids,
blocks and parameter order are those of the reference's engine
(crates/oxide-infer-server/src/batch_engine.rs, "BE" below).  Tensors are
torch CUDA tensors; work is enqueued on torch's current stream.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")

NQ, NKV, HD, KV_DIM, HIDDEN = 16, 4, 128, 512, 2048
CHUNK_KEYS = 128  # BE:49


def available() -> bool:
    return os.path.exists(os.path.join(REF_DIR, "BATCHED_GQA_ATTENTION_SPLIT4_PTX.cubin"))


class RefPtx:
    """Entry-name lookup in modules loaded from the prebuilt cubins (ptx.rs:13-26)."""

    _ENTRIES = {
        "batched_qk_rmsnorm_fp16": "BATCHED_QK_RMSNORM_PTX",
        "batched_rope_fp16": "BATCHED_ROPE_PTX",
        "batched_kv_copy_fp16": "BATCHED_KV_COPY_PTX",
        "batched_gqa_attention_online_fp16": "BATCHED_GQA_ATTENTION_ONLINE_PTX",
        "batched_gqa_attention_split_fp16": "BATCHED_GQA_ATTENTION_SPLIT_PTX",
        "batched_gqa_attn_combine_fp16": "BATCHED_GQA_ATTENTION_SPLIT_PTX",
        "batched_gqa_attention_split4_fp16": "BATCHED_GQA_ATTENTION_SPLIT4_PTX",
        "batched_sigmoid_gate_fp16": "BATCHED_SIGMOID_GATE_PTX",
        "batched_fused_causal_conv1d_gating_ptr_fp16": "BATCHED_CONV_PTR_PTX",
        "conv_state_prefill_fp16": "CONV_STATE_PREFILL_PTX",
        "batched_attn_pack_q_fp16": "BATCHED_ATTN_PACK_Q_PTX",
        "batched_attn_softmax_mask_fp16": "BATCHED_ATTN_SOFTMAX_MASK_PTX",
        "batched_attn_gate_scatter_fp16": "BATCHED_ATTN_GATE_SCATTER_PTX",
        "batched_embed_lookup_fp16": "BATCHED_EMBED_LOOKUP_PTX",
        "batched_argmax_direct_f16": "BATCHED_ARGMAX_DIRECT_PTX",
    }

    def __init__(self):
        from cuda.bindings import driver

        self.drv = driver
        if not available():
            raise RuntimeError("oracle/_ref cubins missing: run python oracle/build_ref.py")
        torch.cuda.init()
        torch.zeros(1, device="cuda")  # make the primary context current
        self._mods = {}
        self._fns = {}
        for entry, const in self._ENTRIES.items():
            if const not in self._mods:
                data = open(os.path.join(REF_DIR, const + ".cubin"), "rb").read()
                err, mod = driver.cuModuleLoadData(data)
                self._chk(err, "cuModuleLoadData " + const)
                self._mods[const] = mod
            err, fn = driver.cuModuleGetFunction(self._mods[const], entry.encode())
            self._chk(err, "cuModuleGetFunction " + entry)
            self._fns[entry] = fn

    def _chk(self, err, what):
        if int(err) != 0:
            raise RuntimeError(f"{what}: CUresult {int(err)}")

    def launch(self, entry, grid, block, args):
        """args: list of (ctype, value); torch tensors are passed as their data pointer."""
        vals, types = [], []
        for t, v in args:
            if isinstance(v, torch.Tensor):
                v = v.data_ptr()
            vals.append(v)
            types.append(t)
        stream = torch.cuda.current_stream().cuda_stream
        (err,) = self.drv.cuLaunchKernel(self._fns[entry], grid[0], grid[1], grid[2], block[0],
                                         block[1], block[2], 0, stream,
                                         (tuple(vals), tuple(types)), 0)
        self._chk(err, "cuLaunchKernel " + entry)

    # ---- operators, launched as the engine launches them ----

    def qk_rmsnorm(self, x_io, w, heads, batch, eps=1e-5):  # BE:941-961
        self.launch("batched_qk_rmsnorm_fp16", (heads, batch, 1), (32, 1, 1),
                    [(C.c_void_p, x_io), (C.c_void_p, w), (C.c_float, eps), (C.c_uint32, heads),
                     (C.c_uint32, HD), (C.c_uint32, batch)])

    def rope(self, x_io, cos, sin, pos_ids, heads, batch):  # BE:963-989
        self.launch("batched_rope_fp16", (heads, batch, 1), (HD, 1, 1),
                    [(C.c_void_p, x_io), (C.c_void_p, cos), (C.c_void_p, sin), (C.c_void_p, pos_ids),
                     (C.c_uint32, heads), (C.c_uint32, HD), (C.c_uint32, batch)])

    def kv_copy(self, dst_ptrs, src, pos_ids, batch):  # BE:991-1014
        self.launch("batched_kv_copy_fp16", (batch, 1, 1), (64, 1, 1),
                    [(C.c_void_p, dst_ptrs), (C.c_void_p, src), (C.c_void_p, pos_ids),
                     (C.c_uint32, KV_DIM), (C.c_uint32, batch)])

    def attn_online(self, ctx, q, k_ptrs, v_ptrs, seq_lens, batch, window):  # BE:1214-1221
        self.launch("batched_gqa_attention_online_fp16", (NKV, batch, 1), (HD, 1, 1),
                    [(C.c_void_p, ctx), (C.c_void_p, q), (C.c_void_p, k_ptrs), (C.c_void_p, v_ptrs),
                     (C.c_void_p, seq_lens), (C.c_uint32, NQ), (C.c_uint32, NKV), (C.c_uint32, HD),
                     (C.c_uint32, batch), (C.c_uint32, window)])

    def attn_split(self, q, k_ptrs, v_ptrs, seq_lens, acc, stats, batch, window, nchunks,
                   entry="batched_gqa_attention_split4_fp16"):  # BE:1155-1193
        self.launch(entry, (NKV, batch, nchunks), (HD, 1, 1),
                    [(C.c_void_p, q), (C.c_void_p, k_ptrs), (C.c_void_p, v_ptrs),
                     (C.c_void_p, seq_lens), (C.c_void_p, acc), (C.c_void_p, stats),
                     (C.c_uint32, NQ), (C.c_uint32, NKV), (C.c_uint32, HD), (C.c_uint32, batch),
                     (C.c_uint32, window), (C.c_uint32, CHUNK_KEYS), (C.c_uint32, nchunks)])

    def attn_combine(self, ctx, acc, stats, batch, nchunks):  # BE:1194-1212
        self.launch("batched_gqa_attn_combine_fp16", (NQ, batch, 1), (32, 1, 1),
                    [(C.c_void_p, ctx), (C.c_void_p, acc), (C.c_void_p, stats), (C.c_uint32, NQ),
                     (C.c_uint32, HD), (C.c_uint32, batch), (C.c_uint32, nchunks)])

    def sigmoid_gate(self, ctx_io, gate, batch):  # BE:1226-1239
        self.launch("batched_sigmoid_gate_fp16", (NQ, batch, 1), (HD, 1, 1),
                    [(C.c_void_p, ctx_io), (C.c_void_p, gate), (C.c_uint32, NQ), (C.c_uint32, HD),
                     (C.c_uint32, batch)])

    def embed_lookup(self, out, table, token_ids, hidden, batch):  # BE:765-779
        self.launch("batched_embed_lookup_fp16", (batch, 1, 1), (256, 1, 1),
                    [(C.c_void_p, out), (C.c_void_p, table), (C.c_void_p, token_ids),
                     (C.c_uint32, hidden), (C.c_uint32, batch)])

    def argmax(self, tokens_out, logits, vocab, batch):  # BE:1367-1378
        self.launch("batched_argmax_direct_f16", (batch, 1, 1), (256, 1, 1),
                    [(C.c_void_p, tokens_out), (C.c_void_p, logits), (C.c_uint32, vocab)])

    def conv_decode(self, y, state_ptrs, bcx, conv_w, batch):  # BE:840-899
        self.launch("batched_fused_causal_conv1d_gating_ptr_fp16", (HIDDEN // 128, batch, 1),
                    (128, 1, 1),
                    [(C.c_void_p, y), (C.c_void_p, state_ptrs), (C.c_void_p, bcx),
                     (C.c_void_p, conv_w), (C.c_uint32, HIDDEN), (C.c_uint32, 7),
                     (C.c_uint32, batch)])

    def conv_state_prefill(self, pool, carry_tbl, origin, local_pos, bcx, rows):  # BE:847-886
        self.launch("conv_state_prefill_fp16", (HIDDEN // 128, rows, 1), (128, 1, 1),
                    [(C.c_void_p, pool), (C.c_void_p, carry_tbl), (C.c_void_p, origin),
                     (C.c_void_p, local_pos), (C.c_void_p, bcx), (C.c_uint32, HIDDEN),
                     (C.c_uint32, 7), (C.c_uint32, rows), (C.c_uint32, HIDDEN * 6),
                     (C.c_uint32, 3 * HIDDEN * 2), (C.c_uint32, 2 * HIDDEN * 2)])

    # ---- the three kernels of the GEMM prefill path (BE:439-592); the two GEMMs between them run in
    # cuBLASLt in the engine and are supplied by the caller

    def attn_pack_q(self, q_pack, q_in, rows):  # BE:477-497: [row][head][dim] -> [head][row][dim]
        self.launch("batched_attn_pack_q_fp16", (rows, 1, 1), (256, 1, 1),
                    [(C.c_void_p, q_in), (C.c_void_p, q_pack), (C.c_uint32, NQ), (C.c_uint32, HD),
                     (C.c_uint32, rows)])

    def attn_softmax_mask(self, scores, p_out, sums, seq_lens, rows, keys, t_lo, window,
                          scale=0.0883883476):  # BE:530-553: one KV head's [4*rows][keys] f32 scores
        self.launch("batched_attn_softmax_mask_fp16", (rows, 4, 1), (128, 1, 1),
                    [(C.c_void_p, scores), (C.c_void_p, p_out), (C.c_void_p, sums), (C.c_void_p, seq_lens),
                     (C.c_uint32, rows), (C.c_uint32, keys), (C.c_uint32, t_lo), (C.c_uint32, window),
                     (C.c_float, scale)])

    def attn_gate_scatter(self, ctx, attn_tmp, gate, sums, rows):  # BE:566-588
        self.launch("batched_attn_gate_scatter_fp16", (NQ, rows, 1), (HD, 1, 1),
                    [(C.c_void_p, ctx), (C.c_void_p, attn_tmp), (C.c_void_p, gate), (C.c_void_p, sums),
                     (C.c_uint32, rows), (C.c_uint32, NQ), (C.c_uint32, HD)])

    def gemm_attention_chunk(self, ctx, q, gate, k_cache, v_cache, seq_lens, rows, slen_min, slen_max, window):
        """BatchEngine::gemm_attention_chunk (BE:439-592) with the two cuBLASLt calls (f16 in, f32
        accumulate) replaced by torch float32 matmuls on the same f16 operands: QK^T to f32 scores,
        PV rounded to f16.  k_cache / v_cache [tokens][4][128] of the chunk's request; seq_lens [rows]
        device u32.  Returns (sums [16][rows] f32) beside writing ctx [rows][16][128]."""
        prev = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = False
        try:
            t_lo = max(slen_min - window, 0) if window > 0 else 0
            keys = slen_max - t_lo
            n = 4 * rows
            qpack = torch.empty(NQ, rows, HD, dtype=torch.float16, device=q.device)
            self.attn_pack_q(qpack, q, rows)
            sums = torch.zeros(NQ * rows, dtype=torch.float32, device=q.device)
            tmp = torch.empty(NQ, rows, HD, dtype=torch.float16, device=q.device)
            for kvh in range(NKV):
                kk = k_cache[t_lo:t_lo + keys, kvh].float()          # [keys][128]
                vv = v_cache[t_lo:t_lo + keys, kvh].float()
                scores = (qpack[4 * kvh:4 * kvh + 4].reshape(n, HD).float() @ kk.t()).contiguous()   # [4*rows][keys]
                p = torch.empty(n, keys, dtype=torch.float16, device=q.device)
                self.attn_softmax_mask(scores, p, sums[kvh * n:(kvh + 1) * n], seq_lens, rows, keys, t_lo, window)
                tmp[4 * kvh:4 * kvh + 4] = (p.float() @ vv).half().view(4, rows, HD)
            self.attn_gate_scatter(ctx, tmp, gate, sums, rows)
            return sums.view(NQ, rows)
        finally:
            torch.backends.cuda.matmul.allow_tf32 = prev

    # ---- the engine's sequences ----

    @staticmethod
    def nchunks_for(max_slen: int, window: int) -> int:
        """BE:1033-1040 without the 64-chunk clamp (the runner sizes partials itself)."""
        eff = min(max_slen, window) if window > 0 else max_slen
        return max(1, -(-eff // CHUNK_KEYS))

    def decode_attention(self, ctx, q, gate, k_ptrs, v_ptrs, seq_lens, batch, window, max_slen,
                         acc=None, stats=None):
        """split4 + combine (or online when one chunk) + gate: BE:1154-1239."""
        nchunks = self.nchunks_for(max_slen, window)
        if nchunks > 1:
            if acc is None:
                acc = torch.empty(batch * nchunks * NQ * HD, dtype=torch.float32, device=q.device)
                stats = torch.empty(batch * nchunks * NQ * 2, dtype=torch.float32, device=q.device)
            self.attn_split(q, k_ptrs, v_ptrs, seq_lens, acc, stats, batch, window, nchunks)
            self.attn_combine(ctx, acc, stats, batch, nchunks)
        else:
            self.attn_online(ctx, q, k_ptrs, v_ptrs, seq_lens, batch, window)
        if gate is not None:
            self.sigmoid_gate(ctx, gate, batch)

    def append(self, q_io, k_io, v_in, q_norm_w, k_norm_w, cos, sin, pos_ids, k_ptrs, v_ptrs,
               batch, eps=1e-5):
        """norm q, norm k, rope q, rope k, copy k, copy v: BE:941-1014 (6 launches)."""
        self.qk_rmsnorm(q_io, q_norm_w, NQ, batch, eps)
        self.qk_rmsnorm(k_io, k_norm_w, NKV, batch, eps)
        self.rope(q_io, cos, sin, pos_ids, NQ, batch)
        self.rope(k_io, cos, sin, pos_ids, NKV, batch)
        self.kv_copy(k_ptrs, k_io, pos_ids, batch)
        self.kv_copy(v_ptrs, v_in, pos_ids, batch)

    def conv_prefill_wave(self, y, pool, carry_tbl, origin, local_pos, bcx, conv_w, rows,
                          carry_host, origin_host):
        """Gather, conv on pool rows, copy each chunk's last pool row back to the request's
        persistent state (BE:847-899 + server.rs:1192-1224)."""
        self.conv_state_prefill(pool, carry_tbl, origin, local_pos, bcx, rows)
        pool_ptrs = torch.tensor([pool.data_ptr() + r * HIDDEN * 6 * 2 for r in range(rows)],
                                 dtype=torch.int64, device=bcx.device)
        self.conv_decode(y, pool_ptrs, bcx, conv_w, rows)
        flat = pool.view(-1)
        for r in range(rows):
            if r + 1 == rows or origin_host[r + 1] != origin_host[r]:
                carry_host[r].view(-1).copy_(flat[r * HIDDEN * 6:(r + 1) * HIDDEN * 6])
