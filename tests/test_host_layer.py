"""Compiles and runs the C++ tests of the host layer (oxide_infer_b200/csrc/host/kv_host.hpp)."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CPP = os.path.join(ROOT, "tests", "cpp")
BUILD = os.path.join(CPP, "build")


def _gxx():
    return "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"


def test_host_layer_allocator_and_tables_cpu():
    os.makedirs(BUILD, exist_ok=True)
    exe = os.path.join(BUILD, "test_kv_host_cpu")
    subprocess.run([_gxx(), "-std=c++17", "-O1", "-Wall", "-o", exe, os.path.join(CPP, "test_kv_host_cpu.cpp")], check=True)
    r = subprocess.run([exe], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "passed" in r.stdout


@pytest.mark.gpu
def test_host_layer_decode_step_gpu():
    from oxide_infer_b200 import build
    so = build.build()
    os.makedirs(BUILD, exist_ok=True)
    exe = os.path.join(BUILD, "test_kv_host_gpu")
    subprocess.run(["nvcc", "-std=c++17", "-O1", "-gencode", "arch=compute_100a,code=sm_100a", "-o", exe,
                    os.path.join(CPP, "test_kv_host_gpu.cpp"), so, "-Xlinker", "-rpath", "-Xlinker",
                    os.path.dirname(so)], check=True)
    r = subprocess.run([exe], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "passed" in r.stdout


@pytest.mark.gpu
def test_host_layer_prefill_waves_equal_token_by_token_decode_gpu():
    """Prompts prefilled in waves planned by the host layer leave the same K/V rows, conv outputs and
    conv states as the same tokens fed one at a time through the decode path."""
    from oxide_infer_b200 import build
    so = build.build()
    os.makedirs(BUILD, exist_ok=True)
    exe = os.path.join(BUILD, "test_kv_host_prefill_gpu")
    subprocess.run(["nvcc", "-std=c++17", "-O1", "-gencode", "arch=compute_100a,code=sm_100a", "-o", exe,
                    os.path.join(CPP, "test_kv_host_prefill_gpu.cpp"), so, "-Xlinker", "-rpath", "-Xlinker",
                    os.path.dirname(so)], check=True)
    r = subprocess.run([exe], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "passed" in r.stdout


@pytest.mark.gpu
def test_host_layer_paged_decode_equals_contiguous_decode_gpu():
    """Decode steps over blocks handed out by the host layer's block manager give the same context bytes
    as the same steps over contiguous leases."""
    from oxide_infer_b200 import build
    so = build.build()
    os.makedirs(BUILD, exist_ok=True)
    exe = os.path.join(BUILD, "test_kv_host_paged_gpu")
    subprocess.run(["nvcc", "-std=c++17", "-O1", "-gencode", "arch=compute_100a,code=sm_100a", "-o", exe,
                    os.path.join(CPP, "test_kv_host_paged_gpu.cpp"), so, "-Xlinker", "-rpath", "-Xlinker",
                    os.path.dirname(so)], check=True)
    r = subprocess.run([exe], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "passed" in r.stdout
