"""Sanitizer substitute: a subset of the parity tests against the bounds-checking build.

liboxi_kv_bounds.so is the same source compiled with -DOXI_BOUNDS: every table-driven index
(cache rows a stage copies, the appended row, partial-result slots, conv chunk positions) is
checked on the device and an index out of range is recorded as OXI_DEV_OUT_OF_BOUNDS instead of
being used.  The parity tests assert a clean status word at fixture teardown, so running them
against this build shows that no such index occurs on the decode edge lengths, the config-2 shape,
the long-row merges, the prefill chunk shapes, the conv paths, the paged layout, the projection GEMM and the
host-buffer step.  A child
process is used because the library path is fixed when the binding is first loaded."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

SUBSET = ("test_decode_config1 or test_decode_edges or test_decode_ragged_batch128 or test_fused_append or "
          "test_decode_long or test_prefill_attn or test_conv or test_append_bit_exact or "
          "test_paged_append or test_paged_fused or test_paged_prefill or test_split or test_project_append or "
          "test_linear_forward or test_host_buffer")


def test_parity_subset_is_clean_under_the_bounds_build():
    if os.environ.get("OXI_KV_LIB"):
        pytest.skip("already running against a substituted library")
    from oxide_infer_b200 import build
    so = build.build(bounds=True)
    env = dict(os.environ, OXI_KV_LIB=so)
    r = subprocess.run([sys.executable, "-m", "pytest", "-q", "-x", "-m", "gpu", "-k", SUBSET,
                        "tests/test_gpu_parity.py", "tests/test_gpu_paged.py", "tests/test_gpu_prefill_split.py",
                        "tests/test_gpu_project.py", "tests/test_gpu_step_order.py"],
                       cwd=ROOT, env=env, capture_output=True, text=True, timeout=900)
    tail = (r.stdout + r.stderr)[-3000:]
    assert r.returncode == 0, tail
    assert " passed" in r.stdout and "failed" not in r.stdout, tail


def test_bounds_build_reports_its_bit_only_there():
    """The bit is part of the ABI (include/oxi_kv.h) and both builds export the same symbols."""
    import ctypes as C
    from oxide_infer_b200 import build, _lib
    a, b = C.CDLL(build.build()), C.CDLL(build.build(bounds=True))
    for name in _lib.SIGNATURES:
        assert hasattr(a, name) and hasattr(b, name), name
