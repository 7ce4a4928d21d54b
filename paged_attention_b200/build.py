"""In-tree build of libpd_b200.so (sm_100a only) with nvcc.

    python -m paged_attention_b200.build [--force]

The library is the product: there is no fallback path, importing the package
without it raises.

Tuning builds: extra nvcc flags come from the environment variable PD_B200_NVCC_FLAGS
(e.g. -DPD_B200_FP8_SHAPE=4222 for another CTA shape of the e4m3 kernel) and
`-o PATH` writes the library somewhere else; PD_B200_LIB points the package at it.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libpd_b200.so")
SOURCES = [os.path.join(CSRC, "pd_abi.cu")]
DEPS = SOURCES + [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(ROOT, "include", "pd_b200.h")]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--use_fast_math",
    "-Xcompiler", "-fPIC", "-shared",
]


def nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    raise RuntimeError("nvcc not found")


def stale():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    return any(os.path.getmtime(d) > t for d in DEPS)


def build(force=False, verbose=False, out=None):
    if not force and not out and not stale():
        return LIB
    extra = os.environ.get("PD_B200_NVCC_FLAGS", "").split()
    cmd = [nvcc()] + NVCC_FLAGS + extra + ["-I" + os.path.join(ROOT, "include"), "-I" + CSRC, "-o", out or LIB] + SOURCES
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
        print(" ".join(cmd))
    subprocess.check_call(cmd)
    return out or LIB


if __name__ == "__main__":
    target = sys.argv[sys.argv.index("-o") + 1] if "-o" in sys.argv else None
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv, out=target))
