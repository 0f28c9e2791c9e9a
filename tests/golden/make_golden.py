"""Generates tests/golden/hotpath_small.npz: seeded inputs of the hot path with the CPU oracle's outputs.

The reference ships no stored vectors for this path (its tests regenerate inputs from a third-party RNG),
and it cannot be built or run where this project is developed, so these fixtures pin the *oracle* (and,
through it, the CUDA kernels) against silent drift; they are not outputs of the reference itself.

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle  # noqa: E402


def main():
    rng = np.random.default_rng(20261125)
    out = {}
    # quantizers: weights ~ N(0, 0.02^2) and the reference tests' 10 * (U - 0.5)
    w = (rng.standard_normal((48, 256), dtype=np.float32) * 0.02).astype(np.float16)
    u = (10.0 * (rng.random((16, 128), dtype=np.float32) - 0.5)).astype(np.float16)
    out["w"], out["u"] = w, u
    out["w_int8"], out["w_minmax"] = oracle.quantize_mat_int8(w)
    out["u_int8"], out["u_minmax"] = oracle.quantize_mat_int8(u)
    out["w_nf4"], out["w_absmax"] = oracle.quantize_mat_nf4(w)
    out["u_nf4"], out["u_absmax"] = oracle.quantize_mat_nf4(u)
    # matmuls: 3 tokens
    x = rng.standard_normal((3, 256), dtype=np.float32).astype(np.float16)
    out["x"] = x
    for name, kind, q, s in (("int8", oracle.MAT_INT8, out["w_int8"], out["w_minmax"]),
                             ("nf4", oracle.MAT_NF4, out["w_nf4"], out["w_absmax"]), ("fp16", oracle.MAT_FP16, w, None)):
        y = np.zeros((3, 48), dtype=np.float32)
        oracle.matmul(kind, q, s, x, y)
        out[f"y_{name}"] = y
    # WKV v6 and v7: 2 heads, two sequences (lengths 3 and 2), wide cursors
    S, H, T, B = 64, 2, 5, 2
    cursors = oracle.pack_cursors([(0, 0, 3), (1, 3, 2)], wide=True)
    out["cursors"] = cursors
    k, v, r = (rng.standard_normal((T, H, S)).astype(np.float32) * 0.5 for _ in range(3))
    xin = rng.standard_normal((T, H, S)).astype(np.float32)
    wdec = np.exp(-np.exp(rng.uniform(-6, 1, (T, H, S)))).astype(np.float32)
    ufirst = rng.uniform(-1, 1, (H, S)).astype(np.float32)
    state = (rng.standard_normal((B, S + 2, S * H)) * 0.1).astype(np.float32)
    out.update(v6_k=k, v6_v=v, v6_r=r, v6_x=xin, v6_w=wdec, v6_u=ufirst, v6_state=state)
    x6, st6 = xin.copy(), state.copy()
    oracle.time_mix_v56(True, cursors, wdec, ufirst, oracle.View(st6, y=(0, S + 1)), k, v, r, x6, S, H)
    out["v6_y"], out["v6_state_out"] = x6, st6
    r7, w7 = rng.standard_normal((T, H, S)).astype(np.float16), rng.standard_normal((T, H, S)).astype(np.float16)
    kk = rng.standard_normal((T, H, S)).astype(np.float32)
    kk /= np.linalg.norm(kk, axis=-1, keepdims=True)
    n7 = np.stack([rng.standard_normal((T, H, S)), rng.standard_normal((T, H, S)), rng.uniform(0, 1, (T, H, S)),
                   kk]).astype(np.float16)
    x7 = rng.standard_normal((T, H, S)).astype(np.float16)
    out.update(v7_r=r7, v7_w=w7, v7_n=n7, v7_x=x7)
    y7, st7 = x7.copy(), state.copy()
    oracle.time_mix_v7(cursors, oracle.View(st7, y=(0, S + 1)), r7, w7, n7, y7, S, H)
    out["v7_y"], out["v7_state_out"] = y7, st7
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "hotpath_small.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
