"""Ahead-of-time build of libkda_b200.so (sm_100a only) with nvcc.

One shared library, built in-tree next to this file; no JIT, no autotuning, no alternative
back end.  ``python -m kda_b200.build`` rebuilds it.
"""

from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(os.path.dirname(HERE), "csrc")
LIB_PATH = os.path.join(HERE, "libkda_b200.so")
SOURCES = [
    "kda_cabi.cu",
    "kda_recurrent.cu",
    "kda_preops.cu",
    "kda_conv.cu",
    "kda_chunk_fwd.cu",
    "kda_prepare_tc.cu",
    "kda_decode_prep.cu",
    "kda_epilogue.cu",
    "kda_state_tc.cu",
    "kda_chunk_bwd.cu",
    "kda_bwd_chunk_tc.cu",
    "kda_cp.cu",
]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def needs_build() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    deps.append(os.path.join(os.path.dirname(os.path.dirname(HERE)), "include", "kda_b200.h"))
    return any(os.path.getmtime(d) > built for d in deps if os.path.exists(d))


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every kernel for sm_100a into one shared library; returns its path."""
    if not force and not needs_build():
        return LIB_PATH
    objs = []
    procs = []
    os.makedirs(os.path.join(HERE, "_obj"), exist_ok=True)
    for src in SOURCES:
        path = os.path.join(CSRC, src)
        if not os.path.exists(path):
            raise FileNotFoundError(path)
        obj = os.path.join(HERE, "_obj", src.replace(".cu", ".o"))
        objs.append(obj)
        cmd = [_nvcc(), *NVCC_FLAGS, "-c", path, "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)))
    for src, proc in procs:
        out, _ = proc.communicate()
        if verbose or proc.returncode:
            sys.stderr.write(out.decode())
        if proc.returncode:
            raise RuntimeError(f"nvcc failed on {src}")
    subprocess.check_call([_nvcc(), "-shared", "-o", LIB_PATH, *objs, "-lcudart", "-ldl"])
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
