"""The C++ face of the engine: the decode:: headers under paged_attention_b200/include are compiled
with g++ into a small caller (tests/cpp/test_decode_api.cpp) that restates cases of the reference's
own hot-path suite through decode::PagedKVCache, and run on the GPU."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "cpp", "test_decode_api.cpp")
EXE = os.path.join(ROOT, "tests", "cpp", "test_decode_api")
LIBDIR = os.path.join(ROOT, "paged_attention_b200")


def build_cpp_test():
    deps = [SRC, os.path.join(ROOT, "include", "pd_b200.h")] + [
        os.path.join(LIBDIR, "include", f) for f in ("decode/decode_types.hpp", "decode/decode.hpp",
                                                     "decode/paged_kv_cache.hpp", "legacy_interfaces.hpp",
                                                     "paged_decode_backend.hpp")] + [os.path.join(LIBDIR, "libpd_b200.so")]
    if os.path.exists(EXE) and all(os.path.getmtime(EXE) >= os.path.getmtime(d) for d in deps):
        return
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    subprocess.check_call(["g++", "-std=c++20", "-O2", "-I", os.path.join(ROOT, "include"),
                           "-I", os.path.join(LIBDIR, "include"), "-I", os.path.join(cuda, "include"), SRC, "-o", EXE,
                           "-L", LIBDIR, "-lpd_b200", "-L", os.path.join(cuda, "lib64"), "-lcudart",
                           "-Wl,-rpath," + LIBDIR])


def test_cpp_headers_compile_against_the_library(pa):
    build_cpp_test()
    assert os.path.exists(EXE)


@pytest.mark.gpu
def test_cpp_caller_runs(torch_cuda, pa):
    build_cpp_test()
    r = subprocess.run([EXE], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
    assert "all checks passed" in r.stdout
