"""A host for the key-range-sharded forward written in C++ against the C ABI alone (tests/cpp/kv_sharded_host.cpp: no PyTorch, no NCCL,
one process per GPU). Without a GPU: it must compile against include/fmha_mxfp8_abi.h and link against the library (every entry it
uses is declared and exported). With at least two GPUs: it runs, and its ranks' output equals, byte for byte, the same problem run on one
GPU."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")


def _build(tmp_path):
    from amdgpu_rustdsl_b200 import _abi
    lib = _abi.lib_path()
    if shutil.which("g++") is None or not os.path.isfile(os.path.join(CUDA, "include", "cuda_runtime.h")) or not os.path.isfile(lib):
        pytest.skip("needs g++, the CUDA toolkit headers and the built library")
    exe = str(tmp_path / "kv_sharded_host")
    libdir = os.path.dirname(lib)
    cmd = ["g++", "-O2", "-std=c++17", "-Wall", "-Werror", f"-I{ROOT}/include", f"-I{CUDA}/include", f"{ROOT}/tests/cpp/kv_sharded_host.cpp", "-o", exe,
           f"-L{libdir}", "-lfmha_mxfp8_b200", f"-L{CUDA}/lib64", "-lcudart", f"-Wl,-rpath,{libdir}", f"-Wl,-rpath,{CUDA}/lib64"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-2000:]
    return exe


def test_cpp_host_compiles_and_links_against_the_c_abi(tmp_path):
    exe = _build(tmp_path)
    r = subprocess.run([exe, "1"], capture_output=True, text=True)   # one rank is not a sharding: refused before anything touches a GPU
    assert r.returncode == 64 and "usage" in r.stderr


@pytest.mark.gpu
def test_cpp_host_runs_the_key_range_shards_without_pytorch(tmp_path):
    torch = pytest.importorskip("torch")
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least two GPUs")
    exe = _build(tmp_path)
    world = 8 if n >= 8 else 4 if n >= 4 else 2
    r = subprocess.run([exe, str(world), "2048", "8192", "4"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "KV_SHARDED_HOST_OK" in r.stdout and f"world={world}" in r.stdout, (r.stdout[-1000:], r.stderr[-2000:])
