"""Builds the same-box GPU comparator oracle/_ref/libqf_ref_gemv.so: this repository's wrapper
(oracle/ref_gpu_launch.cu) around the REFERENCE project's kernel headers, compiled for sm_100a with
the reference's own compiler flags (qfactory/jit/compiler.py:72-77 of the reference), the headers
taken from where they lie under the reference checkout (nothing is copied into this repository).

    python oracle/build_ref.py [/path/to/reference]

Without a reference checkout it does nothing (the prebuilt library, if any, is used as it is).
Test / measurement infrastructure only.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
LIB = os.path.join(OUT_DIR, "libqf_ref_gemv.so")


def build(reference_root: str = "/root/reference", force: bool = False) -> str | None:
    inc = os.path.join(reference_root, "qfactory", "include")
    src = os.path.join(HERE, "ref_gpu_launch.cu")
    if not os.path.exists(os.path.join(inc, "gptq_gemv.h")):
        return LIB if os.path.exists(LIB) else None
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= os.path.getmtime(src):
        return LIB
    os.makedirs(OUT_DIR, exist_ok=True)
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc, "-std=c++20", "-shared", "-O3", "--expt-relaxed-constexpr", "-gencode=arch=compute_100a,code=sm_100a",
           "--compiler-options=-fPIC,-O3", "-I", inc, src, "-o", LIB + ".tmp"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("the reference kernel did not compile for sm_100a")
    os.replace(LIB + ".tmp", LIB)
    return LIB


if __name__ == "__main__":
    print(build(*(sys.argv[1:2] or ["/root/reference"]), force="--force" in sys.argv))
