"""In-tree build of libnimllm_attn.so (sm_100a only) with nvcc.

The library is the product: a C-ABI shared object with no Python or torch types in its
interface.  It is built next to this file so that it ships with the source tree.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libnimllm_attn.so")
SOURCES = ["abi.cu", "rope_append.cu", "decode.cu", "prefill_f32.cu", "prefill_tc.cu", "prefill_bwd.cu", "legacy_abi.cu", "peer.cu", "matvec.cu", "kvpool.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the attention library cannot be built")


def _digest(paths: list[str]) -> str:
    """Content hash of the inputs of one object file (robust against copied trees whose
    modification times no longer order sources before outputs)."""
    h = hashlib.sha256(" ".join(NVCC_FLAGS).encode())
    for p in sorted(paths):
        with open(p, "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def _stale(target: str, deps: list[str]) -> bool:
    stamp = target + ".sha"
    if not os.path.exists(target) or not os.path.exists(stamp):
        return True
    return open(stamp).read().strip() != _digest(deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every .cu file for sm_100a and link libnimllm_attn.so. Returns its path."""
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers.append(os.path.join(HERE, "..", "include", "nimllm_attn.h"))
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    objs, procs = [], []
    for s in SOURCES:
        src = os.path.join(CSRC, s)
        obj = os.path.join(objdir, s.replace(".cu", ".o"))
        objs.append(obj)
        if force or _stale(obj, [src] + headers):
            cmd = [_nvcc(), *NVCC_FLAGS, "-c", src, "-o", obj]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            procs.append((s, obj, [src] + headers,
                          subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for s, obj, deps, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode:
            sys.stderr.write(f"--- {s}\n{out}\n")
        if p.returncode == 0:
            with open(obj + ".sha", "w") as f:
                f.write(_digest(deps))
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    if force or procs or not os.path.exists(LIB):
        subprocess.check_call([_nvcc(), "-shared", "-o", LIB, *objs, "-lcudart"])
    build_host(force or bool(procs))
    return LIB


HOST_LIB = os.path.join(HERE, "libnimllm_attn_host.so")


def build_host(force: bool = False) -> str:
    """The C++ host mirror (nimllm_b200/host): plain C++ over the C ABI, linked against the
    kernel library next to it."""
    srcs = [os.path.join(HERE, "host", "attn_host.cpp")]
    deps = srcs + [os.path.join(HERE, "host", "attn_host.hpp"), os.path.join(HERE, "..", "include", "nimllm_attn.h")]
    if force or _stale(HOST_LIB, deps):
        subprocess.check_call([_nvcc(), "-O2", "-std=c++17", "-Xcompiler", "-fPIC", "-shared", "-o", HOST_LIB, *srcs,
                               "-L" + HERE, "-lnimllm_attn", "-Xlinker", "-rpath=$ORIGIN", "-lcudart"])
        with open(HOST_LIB + ".sha", "w") as f:
            f.write(_digest(deps))
    return HOST_LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
