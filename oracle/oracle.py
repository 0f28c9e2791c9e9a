"""ctypes loader for the CPU oracle (oracle/wrk_oracle.cpp).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the CPU-baseline leg of
bench.py; never by the product package.  Arrays are numpy, shaped (w, z, y, x) for a reference
shape [x, y, z, w]; fp16 data is carried as np.float16, fp32 as np.float32.
"""
import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

ACT_NONE, ACT_SQUARED_RELU, ACT_TANH, ACT_STABLE_EXP, ACT_OPPOSITE_EXP, ACT_SOFTPLUS, ACT_SIGMOID, ACT_SILU = range(8)
MAT_FP16, MAT_INT8, MAT_NF4 = 0, 1, 2

NF4_TABLE = np.array([
    -1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453, -0.28444138169288635,
    -0.18477343022823334, -0.09105003625154495, 0.0, 0.07958029955625534, 0.16093020141124725,
    0.24611230194568634, 0.33791524171829224, 0.44070982933044434, 0.5626170039176941, 0.7229568362236023, 1.0,
], dtype=np.float32)  # src/tensor/matrix.rs:50-67


def sf4_table(nu=5.0):
    """`quantile_student(nu)` of src/tensor/matrix.rs:29-44: Student-t quantiles at 7 probabilities from delta up to
    1/2 and 9 from 1/2 up to 1 - delta, divided by the largest.  The reference takes the quantile from statrs 0.18
    (`StudentsT::inverse_cdf`), which is not part of its tree; scipy's `t.ppf` computes the same function."""
    from scipy import stats
    delta = (1.0 / 32.0 + 1.0 / 30.0) / 2.0
    lo, hi = (0.5 - delta) / 7.0, (1.0 - delta - 0.5) / 8.0
    prob = [delta + lo * i for i in range(7)] + [0.5 + hi * i for i in range(9)]
    q = stats.t.ppf(np.array(prob, dtype=np.float64), nu)
    return (q / q.max()).astype(np.float32)


class _CView(ctypes.Structure):
    _fields_ = [("data", ctypes.c_void_p), ("dtype", ctypes.c_int32), ("shape", ctypes.c_uint32 * 4),
                ("stride", ctypes.c_uint32 * 4), ("offset", ctypes.c_uint32 * 4)]


_libs = {}


def build(fast=False):
    target = "libwrk_oracle_fast.so" if fast else "libwrk_oracle.so"
    subprocess.run(["make", "-C", HERE, target], check=True, stdout=subprocess.DEVNULL)
    return os.path.join(HERE, target)


def lib(fast=False):
    """accuracy build by default; fast=True is the -O3 build used for the timed CPU baseline."""
    if fast not in _libs:
        path = os.path.join(HERE, "libwrk_oracle_fast.so" if fast else "libwrk_oracle.so")
        if not os.path.exists(path):
            build(fast)
        _libs[fast] = ctypes.CDLL(path)
    return _libs[fast]


def _dt(arr):
    if arr.dtype == np.float32:
        return 0
    if arr.dtype == np.float16:
        return 1
    raise TypeError(f"oracle tensors are f32 or f16, got {arr.dtype}")


def _ptr(arr):
    return arr.ctypes.data_as(ctypes.c_void_p)


def ref_shape(arr):
    s = list(arr.shape)[::-1]
    return s + [1] * (4 - len(s))


class View:
    """A view of a numpy array in reference terms: shape / stride / offset over [x, y, z, w]."""

    def __init__(self, arr, x=None, y=None, z=None, w=None):
        assert arr.flags["C_CONTIGUOUS"]
        self.arr = arr
        full = ref_shape(arr)
        self.stride = full
        self.offset, self.shape = [], []
        for dim, r in zip(full, (x, y, z, w)):
            if r is None:
                self.offset.append(0), self.shape.append(dim)
            elif isinstance(r, int):
                self.offset.append(r), self.shape.append(1)
            else:
                self.offset.append(r[0]), self.shape.append(r[1] - r[0])

    def c(self):
        v = _CView()
        v.data = self.arr.ctypes.data
        v.dtype = _dt(self.arr)
        for i in range(4):
            v.shape[i], v.stride[i], v.offset[i] = self.shape[i], self.stride[i], self.offset[i]
        return v


def _view(x):
    return x if isinstance(x, View) else View(x)


def _cursors(cursors):
    """cursors: uint32 array of T packed entries, or (T, 3) wide entries."""
    c = np.ascontiguousarray(cursors, dtype=np.uint32)
    wide = 1 if c.ndim == 2 else 0
    return c, wide


def pack_cursors(cursors, wide=False):
    """[(batch, token, len)] per sequence → per-token cursor array (src/tensor/mod.rs:47-85)."""
    out = []
    for batch, token, length in cursors:
        if length == 0:
            continue
        if wide:
            out += [[batch, token, length]] * length
        else:
            out += [(batch & 0xFF) | ((token & 0xFFFF) << 8) | ((length & 0xFF) << 24)] * length
    if wide:
        return np.array(out, dtype=np.uint32).reshape(-1, 3)
    return np.array(out, dtype=np.uint32)


def quantize_mat_int8(matrix_f16, fast=False):
    m = np.ascontiguousarray(matrix_f16, dtype=np.float16)
    n = m.size
    minmax = np.empty(2 * ((n + 127) // 128), dtype=np.float16)
    out = np.empty(m.shape, dtype=np.uint8)
    lib(fast).orc_quantize_mat_int8(_ptr(m), ctypes.c_uint64(n), _ptr(minmax), _ptr(out))
    return out, minmax


def quantize_mat_nf4(matrix_f16, table=NF4_TABLE, fast=False):
    m = np.ascontiguousarray(matrix_f16, dtype=np.float16)
    n = m.size
    table = np.ascontiguousarray(table, dtype=np.float32)
    absmax = np.empty((n + 63) // 64, dtype=np.float16)
    out = np.empty(m.shape[:-1] + (m.shape[-1] // 2,), dtype=np.uint8)
    lib(fast).orc_quantize_mat_nf4(_ptr(m), ctypes.c_uint64(n), _ptr(table), _ptr(absmax), _ptr(out))
    return out, absmax


def matmul(kind, matrix, scale, input, output, act=ACT_NONE, mode=0, table=NF4_TABLE, fast=False):
    """matrix: (B?, M, K) array (u8 for Int8, packed u8 (…, K/2) for NF4, f16 for fp16)."""
    iv, ov = _view(input), _view(output)
    K = iv.shape[0]
    M = ov.shape[0]
    B = ov.shape[2]
    table = np.ascontiguousarray(table, dtype=np.float32)
    civ, cov = iv.c(), ov.c()
    s = lib(fast).orc_matmul(kind, mode, _ptr(matrix), _ptr(scale) if scale is not None else None, _ptr(table),
                             K, M, B, ctypes.byref(civ), ctypes.byref(cov), act)
    assert s == 0, s


def time_mix_v56(per_token, cursors, time_decay, time_first, state, k, v, r, x, S, H, fast=False):
    c, wide = _cursors(cursors)
    T = x.size // (S * H)
    sv = _view(state).c()
    s = lib(fast).orc_time_mix_v56(int(per_token), _ptr(c), wide, _ptr(time_decay), _ptr(time_first), ctypes.byref(sv),
                                   _dt(x), _ptr(k), _ptr(v), _ptr(r), _ptr(x), S, H, T)
    assert s == 0


def time_mix_v4(cursors, time_decay, time_first, state, k, v, r, x, fast=False):
    """k, v, r, x: (T, C); time_decay, time_first: (C,) f32; state: (B, 4, C) f32 (or a View of it)."""
    c, wide = _cursors(cursors)
    C = x.shape[-1]
    sv = _view(state).c()
    s = lib(fast).orc_time_mix_v4(_ptr(c), wide, _ptr(time_decay), _ptr(time_first), ctypes.byref(sv), _dt(x), _ptr(k),
                                  _ptr(v), _ptr(r), _ptr(x), C, x.size // C)
    assert s == 0


def time_mix_v7(cursors, state, r, w, n, x, S, H, fast=False):
    c, wide = _cursors(cursors)
    T = x.size // (S * H)
    sv = _view(state).c()
    s = lib(fast).orc_time_mix_v7(_ptr(c), wide, ctypes.byref(sv), _dt(x), _ptr(r), _ptr(w), _ptr(n), _ptr(x), S, H, T)
    assert s == 0


def time_first_v7(u, r, n, x, S, H, fast=False):
    T = x.size // (S * H)
    s = lib(fast).orc_time_first_v7(_ptr(u), _dt(x), _ptr(r), _ptr(n), _ptr(x), S, H, T)
    assert s == 0


def layer_norm(w, b, x, eps, fast=False):
    C = x.shape[-1]
    lib(fast).orc_layer_norm(_ptr(w), _ptr(b), _dt(x), _ptr(x), C, x.size // C, 1, ctypes.c_float(eps))


def group_norm(w, b, x, eps, H, fast=False):
    """x: (T, H, S); w, b: (H, S)."""
    S = x.shape[-1]
    lib(fast).orc_layer_norm(_ptr(w), _ptr(b), _dt(x), _ptr(x), S, x.size // S, H, ctypes.c_float(eps))


def softmax(x, fast=False):
    C = x.shape[-1]
    lib(fast).orc_softmax(_dt(x), _ptr(x), C, x.size // C)


def recenter(x, fast=False):
    C = x.shape[-1]
    lib(fast).orc_recenter(_dt(x), _ptr(x), C, x.size // C)


def rms_norm(w, b, x, eps, fast=False):
    C = x.shape[-1]
    lib(fast).orc_rms_norm(_ptr(w), _ptr(b), _dt(x), _ptr(x), C, x.size // C, ctypes.c_float(eps))


def embed(tokens, input, output, fast=False):
    """tokens: (B, T) u32; input: (V, C) f16; output: (B, T, C)."""
    C = output.shape[-1]
    tokens = np.ascontiguousarray(tokens, dtype=np.uint32)
    lib(fast).orc_embed(_ptr(tokens), _ptr(input), _dt(output), _ptr(output), C, output.size // C)


def broadcast(input, output, fast=False):
    iv, ov = _view(input).c(), _view(output).c()
    lib(fast).orc_broadcast(ctypes.byref(iv), ctypes.byref(ov))


def blend(factor, input, output, fast=False):
    factor = np.ascontiguousarray(factor, dtype=np.float32)
    iv, ov = _view(input).c(), _view(output).c()
    lib(fast).orc_blend(_ptr(factor), ctypes.byref(iv), ctypes.byref(ov))


def blend_lora(factor, xa, xb, output, fast=False):
    factor = np.ascontiguousarray(factor, dtype=np.float32)
    av, bv, ov = _view(xa).c(), _view(xb).c(), _view(output).c()
    lib(fast).orc_blend_lora(_ptr(factor), ctypes.byref(av), ctypes.byref(bv), ctypes.byref(ov))


def l2_norm(x, eps, fast=False):
    C = x.shape[-1]
    lib(fast).orc_l2_norm(_dt(x), _ptr(x), C, x.size // C, ctypes.c_float(eps))


def token_shift(cursors, time_mix, state, input, output, reversed, fast=False):
    c, wide = _cursors(cursors)
    tv, sv, ov = _view(time_mix).c(), _view(state).c(), _view(output).c()
    lib(fast).orc_token_shift(_ptr(c), wide, ctypes.byref(tv), ctypes.byref(sv), _dt(input), _ptr(input),
                              ctypes.byref(ov), int(reversed))


def channel_mix(cursors, state, r, v, x, v7=False, fast=False):
    c, wide = _cursors(cursors)
    sv = _view(state).c()
    C = x.shape[-1]
    T = x.size // C
    lib(fast).orc_channel_mix(_ptr(c), wide, ctypes.byref(sv), _dt(x), _ptr(r) if r is not None else None, _ptr(v),
                              _ptr(x), C, T, int(v7))


def binary(is_mul, input, output, act_x=0, act_y=0, act_out=0, fast=False):
    iv, ov = _view(input).c(), _view(output).c()
    lib(fast).orc_binary(int(is_mul), ctypes.byref(iv), ctypes.byref(ov), act_x, act_y, act_out)


def activate(x, act, fast=False):
    xv = _view(x).c()
    lib(fast).orc_activate(ctypes.byref(xv), act)


def blit(input, output, transpose=False, fast=False):
    iv, ov = _view(input).c(), _view(output).c()
    lib(fast).orc_blit(ctypes.byref(iv), ctypes.byref(ov), int(transpose))


def lerp(input, output, factor, reversed, fast=False):
    iv, ov, fv = _view(input).c(), _view(output).c(), _view(factor).c()
    lib(fast).orc_lerp(ctypes.byref(iv), ctypes.byref(ov), ctypes.byref(fv), int(reversed))


def affine(x, scale, bias, fast=False):
    lib(fast).orc_affine(_dt(x), _ptr(x), ctypes.c_uint64(x.size), ctypes.c_float(scale), ctypes.c_float(bias))


def control_k_v7(p, a, k, fast=False):
    av, kv = _view(a).c(), _view(k).c()
    lib(fast).orc_control_k_v7(_ptr(p), ctypes.byref(av), ctypes.byref(kv))


def discount_f16(x, discount):
    x = np.ascontiguousarray(x, dtype=np.float16)
    out = np.empty_like(x)
    lib().orc_discount_f16(_ptr(x), _ptr(out), ctypes.c_uint64(x.size), ctypes.c_float(discount))
    return out


def num_threads(fast=False):
    return lib(fast).orc_num_threads()


def dequant_int8(q, minmax):
    """numpy dequantization fma(q/255, max-min, min) per flat block of 128 (matmul_vec_int8.wgsl:89)."""
    flat = q.reshape(-1).astype(np.float32) / np.float32(255.0)
    mm = minmax.astype(np.float32).reshape(-1, 2)
    mn = np.repeat(mm[:, 0], 128)[: flat.size]
    mx = np.repeat(mm[:, 1], 128)[: flat.size]
    return (flat * (mx - mn) + mn).reshape(q.shape)


def dequant_nf4(packed, absmax, table=NF4_TABLE):
    flat = packed.reshape(-1)
    nib = np.empty(flat.size * 2, dtype=np.uint8)
    nib[0::2] = flat & 15
    nib[1::2] = flat >> 4
    a = np.repeat(absmax.astype(np.float32), 64)[: nib.size]
    return (table[nib] * a).reshape(packed.shape[:-1] + (packed.shape[-1] * 2,))
