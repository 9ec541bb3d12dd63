"""Builds liboxi_kv.so in-tree with nvcc for sm_100a (no other architecture)."""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
SO = os.path.join(HERE, "liboxi_kv.so")
SOURCES = ["oxi_kv.cu", "append_kernels.cu", "decode_attn.cu", "conv_kernels.cu", "prefill_attn.cu", "sample_kernels.cu", "host_api.cu", "stream_probe.cu", "proj_gemm.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "--use_fast_math=false"]


def _stale(so: str = SO) -> bool:
    if not os.path.exists(so):
        return True
    t = os.path.getmtime(so)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cu", ".cuh", ".h", ".hpp"))]
    deps.append(os.path.join(CSRC, "host", "kv_host.hpp"))
    deps.append(os.path.join(HERE, "..", "include", "oxi_kv.h"))
    return any(os.path.getmtime(d) > t for d in deps)


SO_BOUNDS = os.path.join(HERE, "liboxi_kv_bounds.so")


def build(force: bool = False, verbose: bool = False, bounds: bool = False) -> str:
    """bounds=True builds liboxi_kv_bounds.so with -DOXI_BOUNDS: every table-driven index is checked
    and an out-of-range one is recorded in the status word (OXI_DEV_OUT_OF_BOUNDS) instead of being
    used.  The GPU tests run a subset of the parity cases against it (the sanitizer substitute)."""
    so = SO_BOUNDS if bounds else SO
    if not force and not _stale(so):
        return so
    nvcc = os.environ.get("NVCC", "nvcc")
    flags = [f for f in NVCC_FLAGS if not f.startswith("--use_fast_math")]
    if bounds:
        flags.append("-DOXI_BOUNDS")
    objs = []
    for src in SOURCES:
        obj = os.path.join(CSRC, src[:-3] + (".bounds.o" if bounds else ".o"))
        cmd = [nvcc, *flags, "-c", os.path.join(CSRC, src), "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or r.returncode:
            sys.stderr.write(r.stdout + r.stderr)
        if r.returncode:
            raise RuntimeError(f"nvcc failed on {src}")
        objs.append(obj)
    r = subprocess.run([nvcc, "-shared", "-o", so, *objs, "-lcudart"], capture_output=True, text=True)
    if r.returncode:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("link failed")
    return so


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv, bounds="--bounds" in sys.argv))
