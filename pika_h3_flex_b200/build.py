"""Build ``libh3attn.so`` in-tree with nvcc for sm_100a (``python -m pika_h3_flex_b200.build``)."""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "csrc", "h3attn_api.cu")
OUT = os.path.join(HERE, "libh3attn.so")
DEPS = [SRC] + [os.path.join(HERE, "csrc", f) for f in ("attn_fwd.cuh", "attn_fwd_pair.cuh", "qk_prep.cuh", "qkv_proj.cuh", "adaln.cuh", "ptx.cuh")] + [
    os.path.join(HERE, "..", "include", "h3attn.h")
]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
]


def needs_build() -> bool:
    if not os.path.exists(OUT):
        return True
    t = os.path.getmtime(OUT)
    return any(os.path.getmtime(d) > t for d in DEPS)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the library if a source is newer than the binary; return the path of the .so."""
    if not force and not needs_build():
        return OUT
    nvcc = os.environ.get("NVCC", "nvcc")
    cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-o", OUT, SRC, "-lcudart"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("nvcc failed building libh3attn.so")
    if verbose:
        sys.stderr.write(res.stderr)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
