"""Build libb200_paged.so in-tree with nvcc for sm_100a (cross-compiles without a GPU).

    python -m vllm_neuron_b200.build [--force]
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libb200_paged.so")
SOURCES = ["host.cu", "kv_ops.cu", "paged_attn.cu", "paged_attn_prefill_tc.cu", "gemm_tcgen05.cu", "tp_allreduce.cu", "sampling.cu",
           "dyt_norm.cu", "ssm_scan.cu", "swa_attn.cu", "swa_attn_prefill.cu", "swa_attn_prefill_tc.cu", "moe.cu", "rms_norm.cu", "delta_rule.cu",
           "latent_attn.cu", "gated_scan.cu"]
HEADERS = [os.path.join(CSRC, "common.cuh"), os.path.join(CSRC, "hybrid_common.cuh"), os.path.join(os.path.dirname(HERE), "include", "b200_paged.h")]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--threads", "4",
]


def _nvcc() -> str:
    for p in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc"):
        if p and os.path.exists(p):
            return p
    return "nvcc"


def needs_build() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, s) for s in SOURCES] + HEADERS
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not needs_build():
        return LIB
    objs = []
    procs = []
    os.makedirs(os.path.join(HERE, "build"), exist_ok=True)
    newest_header = max(os.path.getmtime(h) for h in HEADERS)
    for s in SOURCES:
        o = os.path.join(HERE, "build", s.replace(".cu", ".o"))
        objs.append(o)
        src = os.path.join(CSRC, s)
        if not force and os.path.exists(o) and os.path.getmtime(o) > max(os.path.getmtime(src), newest_header):
            continue  # this object is up to date: only changed sources are recompiled
        cmd = [_nvcc(), *NVCC_FLAGS, "-c", src, "-o", o]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((s, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for s, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode:
            sys.stderr.write(out)
        if p.returncode:
            raise RuntimeError(f"nvcc failed on {s}")
    # static cudart: the library must load on a box without a GPU/driver (symbol check in the CPU tests)
    cmd = [_nvcc(), "-shared", "-o", LIB, *objs, "-cudart", "static", "-gencode", "arch=compute_100a,code=sm_100a"]
    subprocess.check_call(cmd)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
