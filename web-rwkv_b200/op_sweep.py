"""Op-level sweep of the quantized matmul: `Matrix::matmul_op` over weight shapes and token counts.

    python web-rwkv_b200/op_sweep.py                       # Int8 / NF4 / fp16, three shapes, N in {1, 4, 16, 64, 256, 1024}
    python web-rwkv_b200/op_sweep.py --kind int8 --shape 4096,4096 --tokens 1024 --reps 3 --single
    python web-rwkv_b200/op_sweep.py --wkv                 # time_mix_v7 / v6: 64 heads of 64 x 64 f32 state, T = 1 ... 512

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


def run_wkv(ctx, rng, version, H, T, reps):
    """`time_mix_v7` (fp16 r, w, n, x) or `time_mix_v6` (f32 k, v, r, x) on one sequence of T tokens: H heads of
    64 x 64 f32 state.  The state grows stale over the repetitions, which does not change the work."""
    S = 64
    C = S * H
    cursors = ctx.from_numpy(np.array([[0, 0, T]] * T, dtype=np.uint32))  # wide cursors: (batch, token, len) per token
    state = ctx.from_numpy((rng.standard_normal((1, S + 2, C)) * 0.1).astype(np.float32))
    if version == 7:
        f = np.float16
        r = ctx.from_numpy(rng.standard_normal((T, H, S)).astype(f))
        w = ctx.from_numpy(rng.standard_normal((T, H, S)).astype(f))
        kk = rng.standard_normal((T, H, S)).astype(np.float32)
        kk /= np.linalg.norm(kk, axis=-1, keepdims=True)  # the model L2-normalises kk per head
        n = np.stack([rng.standard_normal((T, H, S)), rng.standard_normal((T, H, S)), rng.uniform(0, 1, (T, H, S)), kk])
        x = ctx.from_numpy(rng.standard_normal((T, H, S)).astype(f))
        op = wrk.time_mix_v7(cursors, state.view(y=(0, S + 1)), r, w, ctx.from_numpy(n.astype(f)), x)
        nbytes = 2.0 * C * S * 4 + T * C * 2.0 * 8
    else:
        f = np.float32
        k, v, r, x = (ctx.from_numpy(rng.standard_normal((T, H, S)).astype(f) * 0.5) for _ in range(4))
        decay = ctx.from_numpy(np.exp(-np.exp(rng.uniform(-6, 1, (T, H, S)))).astype(f))
        first = ctx.from_numpy(rng.uniform(-1, 1, (H, S)).astype(f))
        op = wrk.time_mix_v6(cursors, decay, first, state.view(y=(0, S + 1)), k, v, r, x)
        nbytes = 2.0 * C * S * 4 + T * C * 4.0 * 6
    cmd = ctx.encode(wrk.op_list([op]), use_graph=True)
    for _ in range(3):
        cmd.submit()
    ctx.synchronize()
    ctx.timer_start()
    for _ in range(reps):
        cmd.submit()
    us = ctx.timer_stop() * 1e3 / reps
    flops = (10.0 if version == 7 else 7.0) * C * S * T
    print(f"time_mix_v{version} H={H} T={T}: {us:8.1f} us  {us / T:6.2f} us/token  {nbytes / us / 1e3:8.1f} GB/s  "
          f"{flops / us / 1e6:6.2f} TFLOP/s", flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--wkv", action="store_true", help="sweep time_mix_v7 / time_mix_v6 over T instead of the matmuls")
    ap.add_argument("--kind", default="int8,nf4,fp16")
    ap.add_argument("--shape", action="append", help="K,M (repeatable)")
    ap.add_argument("--tokens", default="1,4,16,64,256,1024")
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--matrices", type=int, default=8)
    ap.add_argument("--single", action="store_true")
    args = ap.parse_args()
    shapes = [tuple(int(v) for v in s.split(",")) for s in (args.shape or ["2048,2048", "2560,8960", "4096,4096"])]
    ctx = wrk.Context(0)
    rng = np.random.default_rng(4000)
    if args.wkv:
        for version in (7, 6):
            for T in (1, 2, 8, 32, 64, 128, 256, 512):
                run_wkv(ctx, rng, version, 64, T, args.reps)
        return
    for kind in args.kind.split(","):
        for K, M in shapes:
            for N in (int(v) for v in args.tokens.split(",")):
                run(ctx, rng, kind, K, M, N, args.reps, args.matrices, args.single)


if __name__ == "__main__":
    main()
