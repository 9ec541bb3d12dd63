"""oxi_decode_attn_static: the decode-attention entry point for hosts that cannot
allocate device memory (its scratch is an array inside the library image).

Called straight through the C ABI, twice in a row with different inputs, and
compared with the handle-based oxi_decode_attn on the same inputs.  The second
call checks that nothing the first call left in the shared array leaks into
the next result.  Collected last on purpose (file name), so a run that stops at
the first failure has already exercised every other test."""
import ctypes as C

import numpy as np
import pytest
import torch

from tests.kvcase import NQ, HD, DecodeCase

pytestmark = pytest.mark.gpu

ATTN_TOL = 2e-3


def _static(lib, d, batch, max_seq_len, window, gate=True):
    st = torch.cuda.current_stream().cuda_stream
    return lib.oxi_decode_attn_static(st, d.ctx.data_ptr(), d.q.data_ptr(),
                                      d.gate.data_ptr() if gate else None, d.k_ptrs.data_ptr(),
                                      d.v_ptrs.data_ptr(), d.seq_lens.data_ptr(), batch, max_seq_len, window)


def test_static_entry_matches_handle_entry_twice():
    from oxide_infer_b200 import KvPath, _lib, build
    build.build()
    lib = _lib.load()
    kv = KvPath(0, max_batch=16, max_seq_len=4096, max_prefill_rows=0)
    try:
        # two different batches back to back: long rows (many key ranges, merge kernel) then a
        # mix with single-range rows and a sliding window
        for lens, window, seed in (([4095, 1000, 257, 3000, 64, 2047], 0, 21), ([300, 5, 4095, 255, 256, 700, 31], 256, 22)):
            case = DecodeCase(lens, seed=seed)
            a, b = case.device(), case.device()
            kv.append(a.q, a.k, a.v, a.q_norm_w, a.k_norm_w, a.cos, a.sin, a.pos_ids, a.k_ptrs, a.v_ptrs)
            kv.append(b.q, b.k, b.v, b.q_norm_w, b.k_norm_w, b.cos, b.sin, b.pos_ids, b.k_ptrs, b.v_ptrs)
            kv.decode_attn(a.ctx, a.q, a.gate, a.k_ptrs, a.v_ptrs, a.seq_lens, window)
            rc = _static(lib, b, case.b, 4096, window)
            assert rc == 0, lib.oxi_status_string(rc)
            torch.cuda.synchronize()
            want, got = a.ctx.float().cpu().numpy(), b.ctx.float().cpu().numpy()
            assert np.isfinite(got).all() and np.abs(got).max() > 0
            assert np.abs(got - want).max() <= ATTN_TOL
            assert torch.equal(a.ctx.view(torch.int16), b.ctx.view(torch.int16))  # same kernels, same bytes
        assert kv.device_status() == 0
    finally:
        kv.close()


def test_static_entry_rejects_sizes_beyond_its_array():
    from oxide_infer_b200 import _lib, build
    build.build()
    lib = _lib.load()
    case = DecodeCase([10, 20], seed=3)
    d = case.device()
    assert _static(lib, d, 17, 4096, 0) == -2          # more rows than the array holds
    assert _static(lib, d, 0, 4096, 0) == -2
    assert _static(lib, d, 2, 4097, 0) == -3           # longer rows than the array holds
    assert _static(lib, d, 2, 0, 0) == -3
    st = torch.cuda.current_stream().cuda_stream
    assert lib.oxi_decode_attn_static(st, None, d.q.data_ptr(), None, d.k_ptrs.data_ptr(),
                                      d.v_ptrs.data_ptr(), d.seq_lens.data_ptr(), 2, 4096, 0) == -1
    before = d.ctx.clone()
    # a row longer than the promised bound is skipped, the other row is computed
    assert _static(lib, d, 2, 16, 0) == 0
    torch.cuda.synchronize()
    assert torch.equal(d.ctx[1], before[1]) and d.ctx[0].abs().sum().item() > 0
    # the skipped row is reported through the path's own status word, which a later call does not clear
    assert _static(lib, d, 1, 16, 0) == 0
    bits = C.c_uint32(0)
    assert lib.oxi_static_device_status(st, C.byref(bits)) == 0
    assert bits.value == 2  # OXI_DEV_BAD_SEQ_LEN
    assert lib.oxi_static_device_status(st, C.byref(bits)) == 0 and bits.value == 0
