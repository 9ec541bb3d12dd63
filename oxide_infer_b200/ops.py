"""Operators of the pointer-table KV-cache path on torch CUDA tensors.

Each function forwards to the C ABI export of the same name (include/oxi_kv.h)
on torch's current stream; torch supplies device memory and streams only.
Argument names and layouts are the reference's (batch_engine.rs launch sites):
``q`` [B,16,128], ``k``/``v`` [B,4,128], ``gate`` [B,16], fp16; ``k_ptrs`` /
``v_ptrs`` / ``conv_ptrs`` int64 device tables of per-sequence device pointers;
``pos_ids`` / ``seq_lens`` int32 device tensors (bit patterns of u32).
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib


class PagedLayout(C.Structure):
    """oxi_paged_layout of include/oxi_kv.h: one layer's K/V pools and the rows' block tables."""
    _fields_ = [("k_pool", C.c_void_p), ("v_pool", C.c_void_p), ("block_tables", C.c_void_p),
                ("block_stride_bytes", C.c_uint64), ("max_blocks", C.c_uint32), ("block_size", C.c_uint32),
                ("num_blocks", C.c_uint32)]

    @classmethod
    def of(cls, k_pool: torch.Tensor, v_pool: torch.Tensor, block_tables: torch.Tensor, block_size: int,
           block_stride_bytes: int | None = None, num_blocks: int | None = None) -> "PagedLayout":
        """k_pool / v_pool [num_blocks][block_size][4][128] f16 (or views with the given stride),
        block_tables [batch][max_blocks] int32."""
        if not block_tables.is_contiguous():
            raise ValueError("block_tables must be contiguous")
        stride = block_stride_bytes if block_stride_bytes is not None else k_pool.stride(0) * k_pool.element_size()
        nb = num_blocks if num_blocks is not None else k_pool.shape[0]
        out = cls(k_pool.data_ptr(), v_pool.data_ptr(), block_tables.data_ptr(), stride, block_tables.shape[1],
                  block_size, nb)
        out._keep = (k_pool, v_pool, block_tables)
        return out


class Linear:
    """Tensor maps over projection weights (oxi_qkvg_create / oxi_linear_create).  The weight tensors are
    kept alive by the object."""

    def __init__(self, *weights):
        lib = _lib.load()
        h = C.c_void_p()
        for w in weights:
            if not (w.is_cuda and w.dtype == torch.float16 and w.is_contiguous() and w.shape[-1] == 2048):
                raise ValueError("weights must be contiguous CUDA f16 [out_features][2048]")
        if len(weights) == 4:
            rc = lib.oxi_qkvg_create(C.byref(h), *[w.data_ptr() for w in weights])
        elif len(weights) == 1:
            rc = lib.oxi_linear_create(C.byref(h), weights[0].data_ptr(), weights[0].shape[0])
        else:
            raise ValueError("one weight matrix, or q, k, v, gate")
        if rc != 0:
            raise OxiError(rc, "oxi_linear_create")
        self.h, self.lib, self._keep = h, lib, weights
        self.out_features = sum(w.shape[0] for w in weights)

    def __del__(self):
        if getattr(self, "h", None):
            self.lib.oxi_linear_destroy(self.h)
            self.h = None


class OxiError(RuntimeError):
    def __init__(self, code: int, where: str):
        lib = _lib.load()
        msg = lib.oxi_last_error_string().decode() or lib.oxi_status_string(code).decode()
        super().__init__(f"{where}: status {code}: {msg}")
        self.code = code


def _check(code: int, where: str) -> None:
    if code != 0:
        raise OxiError(code, where)


def _p(t):
    if t is None:
        return None
    if isinstance(t, torch.Tensor):
        if not t.is_contiguous():
            raise ValueError("tensors passed to liboxi_kv must be contiguous")
        return t.data_ptr()
    return t


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


class KvPath:
    """One per device: owns the library workspace (oxi_create / oxi_destroy)."""

    def __init__(self, device: int = 0, max_batch: int = 128, max_seq_len: int = 8192,
                 max_prefill_rows: int = 512):
        self.lib = _lib.load()
        h = C.c_void_p()
        _check(self.lib.oxi_create(C.byref(h), device, max_batch, max_seq_len, max_prefill_rows),
               "oxi_create")
        self.h = h
        self.device = device

    def close(self):
        if getattr(self, "h", None):
            self.lib.oxi_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def workspace_bytes(self) -> int:
        return int(self.lib.oxi_workspace_bytes(self.h))

    def device_status(self) -> int:
        bits = C.c_uint32(0)
        _check(self.lib.oxi_device_status(self.h, _stream(), C.byref(bits)), "oxi_device_status")
        return bits.value

    def arm_wait_fault(self, which: int, stage: int, limit_us: int = 1000):
        """Test support (oxi_debug_arm_wait_fault): the next decode (which=0) or prefill (which=1)
        attention launch, or the next projection GEMM launch (which=2), loses one pipeline stage of
        CTA 0 and its waits last limit_us."""
        _check(self.lib.oxi_debug_arm_wait_fault(self.h, which, stage, limit_us), "oxi_debug_arm_wait_fault")

    def stream_read(self, src, copy_bytes: int = 4096):
        """Measurement support (oxi_debug_stream_read): reads tensor `src` once through the decode
        kernel's bulk-copy pipeline without arithmetic."""
        _check(self.lib.oxi_debug_stream_read(self.h, _stream(), _p(src), src.numel() * src.element_size(), copy_bytes),
               "oxi_debug_stream_read")

    # ---- fused operators
    def append(self, q_io, k_in, v_in, q_norm_w, k_norm_w, cos, sin, pos_ids, k_ptrs, v_ptrs,
               eps: float = 1e-5, batch: int | None = None):
        b = q_io.shape[0] if batch is None else batch
        _check(self.lib.oxi_append(self.h, _stream(), _p(q_io), _p(k_in), _p(v_in), _p(q_norm_w),
                                   _p(k_norm_w), _p(cos), _p(sin), _p(pos_ids), _p(k_ptrs),
                                   _p(v_ptrs), b, eps), "oxi_append")

    def decode_attn(self, ctx_out, q, gate, k_ptrs, v_ptrs, seq_lens, window: int = 0,
                    batch: int | None = None):
        b = q.shape[0] if batch is None else batch
        _check(self.lib.oxi_decode_attn(self.h, _stream(), _p(ctx_out), _p(q), _p(gate),
                                        _p(k_ptrs), _p(v_ptrs), _p(seq_lens), b, window),
               "oxi_decode_attn")

    def append_decode(self, ctx_out, q_io, k_in, v_in, gate, q_norm_w, k_norm_w, cos, sin, pos_ids,
                      seq_lens, k_ptrs, v_ptrs, window: int = 0, eps: float = 1e-5):
        _check(self.lib.oxi_append_decode(self.h, _stream(), _p(ctx_out), _p(q_io), _p(k_in),
                                          _p(v_in), _p(gate), _p(q_norm_w), _p(k_norm_w), _p(cos),
                                          _p(sin), _p(pos_ids), _p(seq_lens), _p(k_ptrs),
                                          _p(v_ptrs), q_io.shape[0], window, eps),
               "oxi_append_decode")

    def project_append(self, qkvg: Linear, x, q_out, gate_out, q_norm_w, k_norm_w, cos, sin, pos_ids, k_ptrs, v_ptrs,
                       raw_out=None, eps: float = 1e-5, rows: int | None = None):
        """q/k/v/gate projections of x [rows][2048] + RMSNorm + RoPE + KV append in one kernel (oxi_project_append)."""
        n = x.shape[0] if rows is None else rows
        _check(self.lib.oxi_project_append(self.h, _stream(), qkvg.h, _p(x), _p(q_out), _p(gate_out), _p(raw_out),
                                           _p(q_norm_w), _p(k_norm_w), _p(cos), _p(sin), _p(pos_ids), _p(k_ptrs),
                                           _p(v_ptrs), n, eps), "oxi_project_append")

    def linear(self, w: Linear, x, y, rows: int | None = None):
        """y = x W^T (oxi_linear_forward)."""
        n = x.shape[0] if rows is None else rows
        _check(self.lib.oxi_linear_forward(self.h, _stream(), w.h, _p(x), _p(y), n), "oxi_linear_forward")

    def advance_step(self, pos_ids, seq_lens, delta: int = 1, batch: int | None = None):
        """pos_ids += delta, seq_lens += delta on the device (graph-capturable)."""
        t = pos_ids if pos_ids is not None else seq_lens
        b = t.shape[0] if batch is None else batch
        _check(self.lib.oxi_advance_step(self.h, _stream(), _p(pos_ids), _p(seq_lens), b, delta), "oxi_advance_step")

    # ---- paged K/V layout (block tables)
    def append_paged(self, q_io, k_in, v_in, q_norm_w, k_norm_w, cos, sin, pos_ids, layout: PagedLayout,
                     eps: float = 1e-5):
        _check(self.lib.oxi_append_paged(self.h, _stream(), _p(q_io), _p(k_in), _p(v_in), _p(q_norm_w),
                                         _p(k_norm_w), _p(cos), _p(sin), _p(pos_ids), C.addressof(layout),
                                         q_io.shape[0], eps), "oxi_append_paged")

    def decode_attn_paged(self, ctx_out, q, gate, layout: PagedLayout, seq_lens, window: int = 0):
        _check(self.lib.oxi_decode_attn_paged(self.h, _stream(), _p(ctx_out), _p(q), _p(gate),
                                              C.addressof(layout), _p(seq_lens), q.shape[0], window),
               "oxi_decode_attn_paged")

    def append_decode_paged(self, ctx_out, q_io, k_in, v_in, gate, q_norm_w, k_norm_w, cos, sin, seq_lens,
                            layout: PagedLayout, window: int = 0, eps: float = 1e-5):
        _check(self.lib.oxi_append_decode_paged(self.h, _stream(), _p(ctx_out), _p(q_io), _p(k_in), _p(v_in),
                                                _p(gate), _p(q_norm_w), _p(k_norm_w), _p(cos), _p(sin),
                                                _p(seq_lens), C.addressof(layout), q_io.shape[0], window, eps),
               "oxi_append_decode_paged")

    def prefill_attn_paged(self, ctx_out, q, gate, layout: PagedLayout, row_seq, seq_lens, window: int = 0,
                           rows: int | None = None):
        n = q.shape[0] if rows is None else rows
        _check(self.lib.oxi_prefill_attn_paged(self.h, _stream(), _p(ctx_out), _p(q), _p(gate), C.addressof(layout),
                                               _p(row_seq), _p(seq_lens), n, window), "oxi_prefill_attn_paged")

    def prefill_attn(self, ctx_out, q, gate, k_ptrs, v_ptrs, seq_lens, window: int = 0,
                     rows: int | None = None):
        n = q.shape[0] if rows is None else rows
        _check(self.lib.oxi_prefill_attn(self.h, _stream(), _p(ctx_out), _p(q), _p(gate),
                                         _p(k_ptrs), _p(v_ptrs), _p(seq_lens), n, window),
               "oxi_prefill_attn")

    def prefill_split_configure(self, min_part_keys: int, slots: int):
        """Key-range split of small prefill waves: waves with fewer (block, KV head) items than SMs cut
        their long blocks into equal key ranges (enough to fill the SMs once, at most 32 per block, none
        shorter than min_part_keys), with `slots` partial results reserved on the handle
        (prefill_split_slot_bytes() each).  On by default (512 keys, SMs / 4 + 3 slots) for handles with
        max_prefill_rows > 0; min_part_keys = 0 or slots = 0 turns it off.  Synchronises."""
        _check(self.lib.oxi_prefill_split_configure(self.h, min_part_keys, slots), "oxi_prefill_split_configure")

    def register_kv_slab(self, slab):
        """K/V rows of prefill attention that lie inside `slab` (a torch tensor, or None to unregister) at a whole
        number of 1024-byte rows from its start are loaded by the TMA unit."""
        if slab is None:
            _check(self.lib.oxi_register_kv_slab(self.h, None, 0), "oxi_register_kv_slab")
        else:
            _check(self.lib.oxi_register_kv_slab(self.h, _p(slab), slab.numel() * slab.element_size()),
                   "oxi_register_kv_slab")

    def prefill_split_slot_bytes(self) -> int:
        return int(self.lib.oxi_prefill_split_slot_bytes())

    def conv_decode(self, y_out, conv_ptrs, bcx, conv_w, batch: int | None = None):
        b = bcx.shape[0] if batch is None else batch
        _check(self.lib.oxi_conv_decode(self.h, _stream(), _p(y_out), _p(conv_ptrs), _p(bcx),
                                        _p(conv_w), b), "oxi_conv_decode")

    def conv_prefill(self, y_out, carry_ptrs, origin, local_pos, bcx, conv_w,
                     rows: int | None = None):
        n = bcx.shape[0] if rows is None else rows
        _check(self.lib.oxi_conv_prefill(self.h, _stream(), _p(y_out), _p(carry_ptrs), _p(origin),
                                         _p(local_pos), _p(bcx), _p(conv_w), n),
               "oxi_conv_prefill")

    # ---- sampling side of a decode step
    def embed_lookup(self, out, table, token_ids, batch: int | None = None):
        """out[b] = table[token_ids[b]] (batched_embed_lookup_fp16; ids beyond the table zero-fill
        the row and set OXI_DEV_BAD_TOKEN)."""
        b = token_ids.shape[0] if batch is None else batch
        _check(self.lib.oxi_embed_lookup(self.h, _stream(), _p(out), _p(table), _p(token_ids),
                                         table.shape[1], table.shape[0], b), "oxi_embed_lookup")

    def argmax(self, tokens_out, logits, batch: int | None = None):
        """tokens_out[b] = argmax of logits[b] with the reference kernel's tie resolution
        (batched_argmax_direct_f16)."""
        b = logits.shape[0] if batch is None else batch
        _check(self.lib.oxi_argmax(self.h, _stream(), _p(tokens_out), _p(logits), logits.shape[1], b),
               "oxi_argmax")

    # ---- unfused operators (reference semantics, one per PTX entry point)
    def qk_rmsnorm(self, x_io, weight, eps: float = 1e-5):
        b, heads = x_io.shape[0], x_io.shape[1]
        _check(self.lib.oxi_qk_rmsnorm(self.h, _stream(), _p(x_io), _p(weight), eps, heads, b),
               "oxi_qk_rmsnorm")

    def rope(self, x_io, cos, sin, pos_ids):
        b, heads = x_io.shape[0], x_io.shape[1]
        _check(self.lib.oxi_rope(self.h, _stream(), _p(x_io), _p(cos), _p(sin), _p(pos_ids), heads,
                                 b), "oxi_rope")

    def kv_copy(self, dst_ptrs, src, pos_ids):
        _check(self.lib.oxi_kv_copy(self.h, _stream(), _p(dst_ptrs), _p(src), _p(pos_ids),
                                    src.shape[0]), "oxi_kv_copy")

    def sigmoid_gate(self, ctx_io, gate):
        _check(self.lib.oxi_sigmoid_gate(self.h, _stream(), _p(ctx_io), _p(gate), ctx_io.shape[0]),
               "oxi_sigmoid_gate")

    # ---- host-buffer entry
    def decode_step_host(self, ctx_host, q_host, k_host, v_host, gate_host, q_norm_w, k_norm_w,
                         cos, sin, pos_ids_host, k_ptrs_host, v_ptrs_host, batch: int, layers: int,
                         window: int = 0, eps: float = 1e-5):
        _check(self.lib.oxi_decode_step_host(self.h, _stream(), _p(ctx_host), _p(q_host),
                                             _p(k_host), _p(v_host), _p(gate_host), _p(q_norm_w),
                                             _p(k_norm_w), _p(cos), _p(sin), _p(pos_ids_host),
                                             _p(k_ptrs_host), _p(v_ptrs_host), batch, layers,
                                             window, eps), "oxi_decode_step_host")
