"""The CPU answer code of the reference's own matmul tests, restated in numpy.

`test_matmul_int8` (src/tensor/ops.rs:2914-3059) and `test_matmul_nf4` (src/tensor/ops.rs:3064-3256) compute,
on the host, the packed matrix, the block scales and the product they then compare the shaders with.  These
functions follow that host code step by step (f32 arithmetic, the same rounding calls, the same left-to-right
f32 sum over k), so they are a second description of rows A-F that does not share a line with
oracle/wrk_oracle.cpp.  The reference draws its inputs from fastrand (a third-party generator that is not in
the tree), so the inputs here come from numpy's PCG64 with the same distributions; the comparisons the tests
make (`is_approx_eps(.., 0.01)`, u8 within +-1, nibbles equal) are applied by tests/test_oracle.py to the
oracle and by tests/test_gpu_matmul.py to the CUDA kernels.

Run as a script to print the checksums of the answers for the two shapes the reference tests use.
"""
import numpy as np

INT8_BLOCK, NF4_BLOCK = 128, 64

# the table literal of test_matmul_nf4 (src/tensor/ops.rs:3096-3113), identical to Matrix's (src/tensor/matrix.rs:50-67)
NF4_QUANT = np.array([
    -1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453, -0.28444138169288635,
    -0.18477343022823334, -0.09105003625154495, 0.0, 0.07958029955625534, 0.16093020141124725,
    0.24611230194568634, 0.33791524171829224, 0.44070982933044434, 0.5626170039176941, 0.7229568362236023, 1.0,
], dtype=np.float32)


def int8_inputs(c, r, t, seed=42):
    """matrix (r, c) f16 and input (t, c) f16, both 10 * (u - 0.5) with u uniform in [0, 1)."""
    rng = np.random.default_rng(seed)
    matrix = (np.float32(10.0) * (rng.random((r, c), dtype=np.float32) - np.float32(0.5))).astype(np.float16)
    x = (np.float32(10.0) * (rng.random((t, c), dtype=np.float32) - np.float32(0.5))).astype(np.float16)
    return matrix, x


def nf4_inputs(c, r, t, seed=42):
    """matrix (r, c) f16 from Box-Muller normals, input (t, c) f16 uniform in [-1, 1)."""
    rng = np.random.default_rng(seed)
    u = np.maximum(rng.random((r, c), dtype=np.float32), np.float32(1e-30))
    v = rng.random((r, c), dtype=np.float32)
    matrix = (np.sqrt(np.float32(-2.0) * np.log(u)) * np.cos(np.float32(2.0 * np.pi) * v)).astype(np.float16)
    x = (np.float32(2.0) * rng.random((t, c), dtype=np.float32) - np.float32(1.0)).astype(np.float16)
    return matrix, x


def _round_half_away(v):
    """f32::round."""
    return np.where(v >= 0, np.floor(v + np.float32(0.5)), np.ceil(v - np.float32(0.5)))


def int8_quantize(matrix):
    """(matrix_u8, min f16, max f16): per block min / max over the f16 values; round((v - min) / (max - min) * 255)."""
    flat = matrix.reshape(-1, INT8_BLOCK)
    mn, mx = flat.min(axis=1), flat.max(axis=1)
    v, lo, hi = flat.astype(np.float32), mn.astype(np.float32)[:, None], mx.astype(np.float32)[:, None]
    with np.errstate(invalid="ignore", divide="ignore"):
        q = _round_half_away((v - lo) / (hi - lo) * np.float32(255.0))
    return np.nan_to_num(q, nan=0.0).astype(np.uint8).reshape(matrix.shape), mn, mx


def _fold(terms):
    """Left-to-right f32 sum over the last axis (Iterator::fold with an f32 accumulator)."""
    return np.add.accumulate(terms.astype(np.float32), axis=-1, dtype=np.float32)[..., -1]


def int8_answer(matrix_u8, mn, mx, x):
    """ans[token][line] = fold over i of (u8 / 255 * (max - min) + min) * x, all in f32."""
    r, c = matrix_u8.shape
    lo = np.repeat(mn.astype(np.float32), INT8_BLOCK).reshape(r, c)  # blocks are flat: (line * c + i) / 128
    hi = np.repeat(mx.astype(np.float32), INT8_BLOCK).reshape(r, c)
    w = matrix_u8.astype(np.float32) / np.float32(255.0) * (hi - lo) + lo
    xf = x.astype(np.float32)
    return np.stack([_fold(w * xf[t][None, :]) for t in range(x.shape[0])])


def nf4_quantize(matrix):
    """(indices u8 (r, c), packed u4 (r, c / 2), absmax f16): value / absmax, first minimum of |value - quant| wins."""
    flat = matrix.reshape(-1, NF4_BLOCK)
    absmax = np.abs(flat).max(axis=1)
    with np.errstate(invalid="ignore", divide="ignore"):
        v = flat.astype(np.float32) / absmax.astype(np.float32)[:, None]
    err = np.abs(v[..., None] - NF4_QUANT[None, None, :])
    # fold((0, f32::MAX), |acc, x| if x.1 < acc.1 { x } else { acc }): NaN never compares below, index stays 0
    idx = np.where(np.isnan(v), 0, np.argmin(np.where(np.isnan(err), np.float32(np.inf), err), axis=-1)).astype(np.uint8)
    idx = idx.reshape(matrix.shape)
    packed = (idx[:, 0::2] | (idx[:, 1::2] << 4)).astype(np.uint8)
    return idx, packed, absmax


def nf4_answer(idx, absmax, x):
    """ans[token][line] = fold over i of quant[u8] * absmax * x in f32."""
    r, c = idx.shape
    amp = np.repeat(absmax.astype(np.float32), NF4_BLOCK).reshape(r, c)  # (line * c + i) / 64
    w = NF4_QUANT[idx] * amp
    xf = x.astype(np.float32)
    return np.stack([_fold(w * xf[t][None, :]) for t in range(x.shape[0])])


def is_approx_eps(a, b, eps):
    """src/tensor/ops.rs:2614-2618."""
    a = np.asarray(a, dtype=np.float32)
    b = np.asarray(b, dtype=np.float32)
    return np.abs(a - b) <= np.maximum(np.float32(eps), np.maximum(np.abs(a), np.abs(b)) * np.float32(eps))


if __name__ == "__main__":
    import zlib
    for c, r, t in ((2560, 2048, 64), (320, 64, 320)):
        m, x = int8_inputs(c, r, t)
        q, mn, mx = int8_quantize(m)
        print("int8", c, r, t, zlib.crc32(q.tobytes()), zlib.crc32(int8_answer(q, mn, mx, x).tobytes()))
        if c % NF4_BLOCK == 0:
            m, x = nf4_inputs(c, r, t)
            idx, packed, am = nf4_quantize(m)
            print("nf4", c, r, t, zlib.crc32(packed.tobytes()), zlib.crc32(nf4_answer(idx, am, x).tobytes()))
