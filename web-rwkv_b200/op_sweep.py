"""Op-level sweep of the quantized matmul: `Matrix::matmul_op` over weight shapes and token counts.

    python web-rwkv_b200/op_sweep.py                       # Int8 / NF4 / fp16, three shapes, N in {1, 16, 64, 256, 1024}
    python web-rwkv_b200/op_sweep.py --kind int8 --shape 4096,4096 --tokens 1024 --reps 3 --single

Each line is the CUDA-event time per launch of a graph that holds `--matrices` different weight matrices of the
shape (so that consecutive launches do not re-read one matrix from L2), the algorithmic bytes per second and the
flops per second.  `--single` submits one op per launch without a graph (the form used under a profiler).
"""
import argparse
import importlib
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
wrk = importlib.import_module("web-rwkv_b200")

BYTES_PER_WEIGHT = {"int8": 1.0 + 4.0 / 128.0, "nf4": 0.5 + 2.0 / 64.0, "fp16": 2.0}


def make_matrix(ctx, kind, rng, K, M):
    w = ctx.from_numpy((rng.standard_normal((M, K), dtype=np.float32) * 0.02).astype(np.float16))
    if kind == "int8":
        return wrk.Matrix.quant_u8(w)
    if kind == "nf4":
        return wrk.Matrix.quant_nf4(w)
    return wrk.Matrix.fp16(w)


def run(ctx, rng, kind, K, M, N, reps, matrices, single):
    mats = [make_matrix(ctx, kind, rng, K, M) for _ in range(1 if single else matrices)]
    x = ctx.from_numpy(rng.standard_normal((N, K), dtype=np.float32).astype(np.float16))
    y = ctx.tensor(wrk.F16, [M, N])
    ops = [m.matmul_op(x, y, turbo=(N % 32 == 0)) for m in mats]
    if single:
        for _ in range(reps):
            ctx.run(ops[0])
        ctx.synchronize()
        print(f"{kind} K={K} M={M} N={N}: {reps} single launches", flush=True)
        return
    cmd = ctx.encode(wrk.op_list(ops), use_graph=True)
    for _ in range(3):
        cmd.submit()
    ctx.synchronize()
    ctx.timer_start()
    for _ in range(reps):
        cmd.submit()
    us = ctx.timer_stop() * 1e3 / (reps * len(mats))
    nbytes = K * M * BYTES_PER_WEIGHT[kind] + 2.0 * N * (K + M)
    print(f"{kind} K={K} M={M} N={N}: {us:8.1f} us  {nbytes / us / 1e3:8.1f} GB/s  {2.0 * K * M * N / us / 1e6:8.1f} TFLOP/s",
          flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--kind", default="int8,nf4,fp16")
    ap.add_argument("--shape", action="append", help="K,M (repeatable)")
    ap.add_argument("--tokens", default="1,16,64,256,1024")
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--matrices", type=int, default=8)
    ap.add_argument("--single", action="store_true")
    args = ap.parse_args()
    shapes = [tuple(int(v) for v in s.split(",")) for s in (args.shape or ["2048,2048", "2560,8960", "4096,4096"])]
    ctx = wrk.Context(0)
    rng = np.random.default_rng(4000)
    for kind in args.kind.split(","):
        for K, M in shapes:
            for N in (int(v) for v in args.tokens.split(",")):
                run(ctx, rng, kind, K, M, N, args.reps, args.matrices, args.single)


if __name__ == "__main__":
    main()
