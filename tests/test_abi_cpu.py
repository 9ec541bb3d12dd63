"""Host-only checks of the C ABI: the library loads, exports every symbol the
header declares, and refuses to create a handle without a device."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from oxide_infer_b200 import build, _lib
    build.build()
    return _lib.load()


def test_header_symbols_are_exported(lib):
    text = open(os.path.join(ROOT, "include", "oxi_kv.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = set(re.findall(r"\b(oxi_[a-z0-9_]+)\s*\(", text))
    assert len(names) >= 18
    from oxide_infer_b200 import _lib
    assert names == set(_lib.SIGNATURES), names ^ set(_lib.SIGNATURES)
    for n in names:
        assert hasattr(lib, n), n


def test_rust_binding_in_the_integration_notes_names_every_export():
    """The `extern "C"` block a maintainer copies declares exactly the header's functions."""
    text = open(os.path.join(ROOT, "include", "oxi_kv.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = set(re.findall(r"\b(oxi_[a-z0-9_]+)\s*\(", text))
    rust = set(re.findall(r"pub fn (oxi_[a-z0-9_]+)\s*\(", open(os.path.join(ROOT, "INTEGRATION.md")).read()))
    assert rust == names, rust ^ names


def test_version_and_status_strings(lib):
    assert lib.oxi_version() == 100
    assert lib.oxi_status_string(0) == b"ok"
    assert b"null" in lib.oxi_status_string(-1)
    assert b"batch" in lib.oxi_status_string(-2)


def test_create_argument_errors_need_no_device(lib):
    h = C.c_void_p()
    assert lib.oxi_create(None, 0, 8, 1024, 0) == -1
    assert lib.oxi_create(C.byref(h), 0, 0, 1024, 0) == -2
    assert lib.oxi_create(C.byref(h), 0, 1025, 1024, 0) == -2
    assert lib.oxi_create(C.byref(h), 0, 8, 0, 0) == -3
    assert h.value is None
    assert lib.oxi_destroy(None) == 0


def test_create_without_gpu_fails_cleanly(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    h = C.c_void_p()
    assert lib.oxi_create(C.byref(h), 0, 8, 1024, 0) == -5
    assert b"device" in lib.oxi_last_error_string()
    # operators reject a null handle before touching CUDA
    assert lib.oxi_append(None, *([None] * 11), 1, 1e-5) == -1
    assert lib.oxi_decode_attn(None, *([None] * 7), 1, 0) == -1
    assert lib.oxi_argmax(None, None, None, None, 128000, 1) == -1
    assert lib.oxi_embed_lookup(None, None, None, None, None, 2048, 128000, 1) == -1
    assert lib.oxi_advance_step(None, None, None, None, 1, 1) == -1
    assert lib.oxi_append_paged(None, *([None] * 10), 1, 1e-5) == -1
    assert lib.oxi_decode_attn_paged(None, *([None] * 6), 1, 0) == -1
    assert lib.oxi_append_decode_paged(None, *([None] * 12), 1, 0, 1e-5) == -1
    assert lib.oxi_prefill_attn_paged(None, *([None] * 7), 1, 0) == -1
    assert lib.oxi_prefill_split_configure(None, 256, 16) == -1
    assert lib.oxi_register_kv_slab(None, None, 0) == -1
    assert lib.oxi_prefill_split_slot_bytes() == 4 * 2 * 128 * 130 * 4


def test_package_has_no_fallback(monkeypatch):
    from oxide_infer_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "SO_PATH", "/nonexistent/liboxi_kv.so")
    with pytest.raises(ImportError):
        _lib.load()
