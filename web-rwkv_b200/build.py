"""Build recipe for libwrk.so (the sm_100a CUDA library behind include/wrk.h).

Run as a script (`python web-rwkv_b200/build.py`) or call `build()`.  The library is built
in-tree, next to this file, with nvcc; no PyTorch is involved.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libwrk.so")
OBJ = os.path.join(HERE, "build")

SOURCES = [
    "context.cpp",
    "ops.cpp",
    "comm.cpp",
    "kernels/quant.cu",
    "kernels/matmul.cu",
    "kernels/gemm_umma.cu",
    "kernels/gemm_small.cu",
    "kernels/wkv.cu",
    "kernels/support.cu",
    "kernels/elementwise.cu",
    "kernels/peer_reduce.cu",
    "kernels/decode.cu",
    "kernels/decode_step.cu",
    "kernels/decode_step_umma.cu",
    "runtime/rnn.cpp",
    "runtime/model.cpp",
    "runtime/bundle.cpp",
    "runtime/serialize.cpp",
]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-ccbin", "/usr/bin/g++",
]


def _nvcc():
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; libwrk.so cannot be built")
    return nvcc


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False, extra_flags=()):
    """Compile every source to an object (only when stale) and link libwrk.so."""
    nvcc = _nvcc()
    os.makedirs(OBJ, exist_ok=True)
    headers = []
    for root, _, files in os.walk(CSRC):
        headers += [os.path.join(root, f) for f in files if f.endswith((".h", ".cuh"))]
    headers.append(os.path.join(HERE, "..", "include", "wrk.h"))
    rt = os.path.join(HERE, "..", "include", "wrk_runtime.h")
    if os.path.exists(rt):
        headers.append(rt)
    objects = []
    procs = []
    for src in SOURCES:
        path = os.path.join(CSRC, src)
        if not os.path.exists(path):
            continue
        obj = os.path.join(OBJ, src.replace("/", "_") + ".o")
        objects.append(obj)
        if force or _stale(obj, [path] + headers):
            cmd = [nvcc, *NVCC_FLAGS, *extra_flags, "-x", "cu", "-c", path, "-o", obj]
            if verbose:
                print(" ".join(cmd), flush=True)
            procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            failed = True
            sys.stderr.write(f"--- {src} ---\n{out}\n")
        elif verbose and out.strip():
            print(out)
    if failed:
        raise RuntimeError("nvcc failed")
    if procs or force or not os.path.exists(LIB):
        cmd = [nvcc, "-shared", "-ccbin", "/usr/bin/g++", "-o", LIB, *objects, "-ldl"]
        subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose=True,
          extra_flags=("-Xptxas", "-v") if "--ptxas" in sys.argv else ())
    print(LIB)
