"""ctypes harness over libwrk.so, the sm_100a library behind include/wrk.h.

This package is the Python-side mirror of the reference crate's operator interface
(`TensorOp`, `Matrix`, tensors and views; src/tensor/ops.rs, src/tensor/matrix.rs) used by the
tests and the benchmark.  It contains no compute of its own and no fallback: every call goes
through the C ABI, and importing `lib()` fails loudly when the CUDA library has not been built.

Shapes follow the reference: ``[x, y, z, w]`` with ``x`` fastest.  A numpy array of shape
``(w, z, y, x)`` (trailing axis fastest) maps to the tensor shape ``[x, y, z, w]``.
"""
import ctypes
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libwrk.so")

F32, F16, U8, U16, U32 = 0, 1, 2, 3, 4
ACT_NONE, ACT_SQUARED_RELU, ACT_TANH, ACT_STABLE_EXP, ACT_OPPOSITE_EXP, ACT_SOFTPLUS, ACT_SIGMOID, ACT_SILU = range(8)
QUANT_NONE, QUANT_INT8, QUANT_NF4, QUANT_SF4 = range(4)
RNN_LAST, RNN_FULL, RNN_NONE = range(3)
DIM_AUTO = 0xFFFFFFFF

_NP = {F32: np.float32, F16: np.float16, U8: np.uint8, U16: np.uint16, U32: np.uint32}
_DT = {np.dtype(v): k for k, v in _NP.items()}


ERR_NCCL, ERR_TIMEOUT, ERR_INVALID_ARGUMENT, ERR_UNSUPPORTED = -101, -102, -103, -104  # wrk_status, include/wrk.h


class WrkError(RuntimeError):
    def __init__(self, status, message):
        super().__init__(f"wrk status {status}: {message}")
        self.status = status
        self.message = message


class CView(ctypes.Structure):
    _fields_ = [("tensor", ctypes.c_void_p), ("shape", ctypes.c_uint32 * 4), ("stride", ctypes.c_uint32 * 4),
                ("offset", ctypes.c_uint32 * 4)]


_lib = None


def lib():
    """The loaded C library.  Raises if libwrk.so is missing: there is no CPU fallback."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} not found: build it with `python web-rwkv_b200/build.py` "
                              "(there is no CPU fallback for the CUDA path)")
        _lib = ctypes.CDLL(LIB_PATH)
        _lib.wrk_last_error_message.restype = ctypes.c_char_p
        _lib.wrk_build_arch.restype = ctypes.c_char_p
    return _lib


def check(status):
    if status != 0:
        raise WrkError(status, lib().wrk_last_error_message().decode())


def _shape4(shape):
    s = list(shape) + [1] * (4 - len(shape))
    return (ctypes.c_uint32 * 4)(*s)


def np_to_shape(arr):
    """numpy (…, y, x) → reference [x, y, z, w]."""
    s = list(arr.shape)[::-1]
    assert len(s) <= 4
    return s + [1] * (4 - len(s))


class Context:
    def __init__(self, device=0):
        self.handle = ctypes.c_void_p()
        check(lib().wrk_context_create(device, ctypes.byref(self.handle)))

    def close(self):
        if self.handle:
            lib().wrk_context_destroy(self.handle)
            self.handle = ctypes.c_void_p()

    def synchronize(self):
        check(lib().wrk_context_synchronize(self.handle))

    def device_status(self):
        s = ctypes.c_int32()
        check(lib().wrk_context_device_status(self.handle, ctypes.byref(s)))
        return s.value

    def launch_count(self):
        n = ctypes.c_uint64()
        check(lib().wrk_context_launch_count(self.handle, ctypes.byref(n)))
        return n.value

    def timer_start(self):
        check(lib().wrk_timer_start(self.handle))

    def timer_stop(self):
        ms = ctypes.c_float()
        check(lib().wrk_timer_stop(self.handle, ctypes.byref(ms)))
        return ms.value

    # tensors
    def tensor(self, dtype, shape, zeros=False):
        h = ctypes.c_void_p()
        fn = lib().wrk_tensor_zeros if zeros else lib().wrk_tensor_create
        check(fn(self.handle, dtype, _shape4(shape), ctypes.byref(h)))
        return Tensor(self, h)

    def from_numpy(self, arr, shape=None):
        arr = np.ascontiguousarray(arr)
        dtype = _DT[arr.dtype]
        shape = np_to_shape(arr) if shape is None else list(shape)
        h = ctypes.c_void_p()
        check(lib().wrk_tensor_from_data(self.handle, dtype, _shape4(shape), arr.ctypes.data_as(ctypes.c_void_p),
                                         ctypes.c_size_t(arr.nbytes), ctypes.byref(h)))
        return Tensor(self, h)

    def run(self, op):
        check(lib().wrk_run(self.handle, op.handle))

    def encode(self, op, use_graph=False):
        h = ctypes.c_void_p()
        check(lib().wrk_encode(self.handle, op.handle, int(use_graph), ctypes.byref(h)))
        return Commands(self, h)


class Commands:
    def __init__(self, ctx, handle):
        self.ctx, self.handle = ctx, handle

    def submit(self):
        check(lib().wrk_submit(self.ctx.handle, self.handle))

    def __del__(self):
        if self.handle and _lib is not None:
            _lib.wrk_commands_release(self.handle)
            self.handle = None


class Tensor:
    def __init__(self, ctx, handle):
        self.ctx, self.handle = ctx, handle

    def __del__(self):
        if getattr(self, "handle", None) and _lib is not None:
            _lib.wrk_tensor_release(self.handle)
            self.handle = None

    @property
    def shape(self):
        s = (ctypes.c_uint32 * 4)()
        check(lib().wrk_tensor_shape(self.handle, s))
        return list(s)

    @property
    def dtype(self):
        d = ctypes.c_int32()
        check(lib().wrk_tensor_dtype(self.handle, ctypes.byref(d)))
        return d.value

    def numpy(self):
        """Read back as a numpy array of shape (w, z, y, x)."""
        shape = self.shape
        arr = np.empty(shape[::-1], dtype=_NP[self.dtype])
        check(lib().wrk_tensor_back(self.handle, arr.ctypes.data_as(ctypes.c_void_p), ctypes.c_size_t(arr.nbytes)))
        return arr

    def load(self, arr):
        arr = np.ascontiguousarray(arr, dtype=_NP[self.dtype])
        check(lib().wrk_tensor_load(self.handle, arr.ctypes.data_as(ctypes.c_void_p), ctypes.c_size_t(arr.nbytes)))

    def reshape(self, x, y=1, z=1, w=1):
        h = ctypes.c_void_p()
        check(lib().wrk_tensor_reshape(self.handle, _shape4([x, y, z, w]), ctypes.byref(h)))
        return Tensor(self.ctx, h)

    def view(self, x=None, y=None, z=None, w=None):
        """Half-open ranges per axis (None = whole axis, int = single index)."""
        shape = self.shape
        start, end = [], []
        for dim, r in zip(shape, (x, y, z, w)):
            if r is None:
                start.append(0), end.append(dim)
            elif isinstance(r, int):
                start.append(r), end.append(r + 1)
            else:
                start.append(r[0]), end.append(r[1])
        v = CView()
        check(lib().wrk_tensor_view(self.handle, _shape4(start), _shape4(end), ctypes.byref(v)))
        return View(self, v)

    def as_view(self):
        v = CView()
        check(lib().wrk_tensor_as_view(self.handle, ctypes.byref(v)))
        return View(self, v)


class View:
    def __init__(self, tensor, cview):
        self.tensor, self.c = tensor, cview  # keeps the tensor alive


def _v(x):
    """Tensor or View → pointer to a wrk_view."""
    if isinstance(x, Tensor):
        x = x.as_view()
    return ctypes.byref(x.c), x


class Op:
    def __init__(self, handle, keep=()):
        self.handle, self.keep = handle, keep

    def __del__(self):
        if self.handle and _lib is not None:
            _lib.wrk_op_release(self.handle)
            self.handle = None

    def num_atoms(self):
        n = ctypes.c_uint64()
        check(lib().wrk_op_num_atoms(self.handle, ctypes.byref(n)))
        return n.value


def _mk(fn_name, *args, keep=()):
    h = ctypes.c_void_p()
    check(getattr(lib(), fn_name)(*args, ctypes.byref(h)))
    return Op(h, keep)


def _t(x):
    return x.handle if x is not None else None


def op_list(ops):
    arr = (ctypes.c_void_p * len(ops))(*[o.handle for o in ops])
    return _mk("wrk_op_list", arr, ctypes.c_size_t(len(ops)), keep=tuple(ops))


def quantize_mat_int8(input, minmax, output):
    return _mk("wrk_op_quantize_mat_int8", _t(input), _t(minmax), _t(output), keep=(input, minmax, output))


def quantize_mat_nf4(input, quant, absmax, output):
    return _mk("wrk_op_quantize_mat_nf4", _t(input), _t(quant), _t(absmax), _t(output),
               keep=(input, quant, absmax, output))


def matmul_vec_fp16(matrix, input, output, act=ACT_NONE, sparse=False):
    (pi, ki), (po, ko) = _v(input), _v(output)
    return _mk("wrk_op_matmul_vec_fp16", _t(matrix), pi, po, act, int(sparse), keep=(matrix, ki, ko))


def matmul_vec_int8(matrix, minmax, input, output, act=ACT_NONE, sparse=False):
    (pi, ki), (po, ko) = _v(input), _v(output)
    return _mk("wrk_op_matmul_vec_int8", _t(matrix), _t(minmax), pi, po, act, int(sparse),
               keep=(matrix, minmax, ki, ko))


def matmul_vec_nf4(matrix, quant, absmax, input, output, act=ACT_NONE, sparse=False):
    (pi, ki), (po, ko) = _v(input), _v(output)
    return _mk("wrk_op_matmul_vec_nf4", _t(matrix), _t(quant), _t(absmax), pi, po, act, int(sparse),
               keep=(matrix, quant, absmax, ki, ko))


def matmul_mat_fp16(matrix, input, output, act=ACT_NONE):
    (pm, km), (pi, ki), (po, ko) = _v(matrix), _v(input), _v(output)
    return _mk("wrk_op_matmul_mat_fp16", pm, pi, po, act, keep=(km, ki, ko))


def matmul_mat_int8(matrix, minmax, input, output, act=ACT_NONE):
    (pm, km), (pi, ki), (po, ko) = _v(matrix), _v(input), _v(output)
    return _mk("wrk_op_matmul_mat_int8", pm, _t(minmax), pi, po, act, keep=(km, minmax, ki, ko))


def matmul_mat_nf4(matrix, quant, absmax, input, output, act=ACT_NONE):
    (pm, km), (pi, ki), (po, ko) = _v(matrix), _v(input), _v(output)
    return _mk("wrk_op_matmul_mat_nf4", pm, _t(quant), _t(absmax), pi, po, act, keep=(km, quant, absmax, ki, ko))


def time_mix_v4(cursors, time_decay, time_first, state, k, v, r, x):
    ps, ks = _v(state)
    return _mk("wrk_op_time_mix_v4", _t(cursors), _t(time_decay), _t(time_first), ps, _t(k), _t(v), _t(r), _t(x),
               keep=(cursors, time_decay, time_first, ks, k, v, r, x))


def time_mix_v5(cursors, time_decay, time_first, state, k, v, r, x):
    ps, ks = _v(state)
    return _mk("wrk_op_time_mix_v5", _t(cursors), _t(time_decay), _t(time_first), ps, _t(k), _t(v), _t(r), _t(x),
               keep=(cursors, time_decay, time_first, ks, k, v, r, x))


def time_mix_v6(cursors, time_decay, time_first, state, k, v, r, x):
    ps, ks = _v(state)
    return _mk("wrk_op_time_mix_v6", _t(cursors), _t(time_decay), _t(time_first), ps, _t(k), _t(v), _t(r), _t(x),
               keep=(cursors, time_decay, time_first, ks, k, v, r, x))


def time_mix_v7(cursors, state, r, w, n, x):
    ps, ks = _v(state)
    return _mk("wrk_op_time_mix_v7", _t(cursors), ps, _t(r), _t(w), _t(n), _t(x), keep=(cursors, ks, r, w, n, x))


def time_first_v7(u, r, n, x):
    return _mk("wrk_op_time_first_v7", _t(u), _t(r), _t(n), _t(x), keep=(u, r, n, x))


def layer_norm(w, b, x, eps):
    return _mk("wrk_op_layer_norm", _t(w), _t(b), _t(x), ctypes.c_float(eps), keep=(w, b, x))


def group_norm(w, b, x, eps):
    return _mk("wrk_op_group_norm", _t(w), _t(b), _t(x), ctypes.c_float(eps), keep=(w, b, x))


def softmax(x):
    return _mk("wrk_op_softmax", _t(x), keep=(x,))


def embed(tokens, input, output):
    return _mk("wrk_op_embed", _t(tokens), _t(input), _t(output), keep=(tokens, input, output))


def recenter(x):
    return _mk("wrk_op_recenter", _t(x), keep=(x,))


def rms_norm(w, b, x, eps):
    return _mk("wrk_op_rms_norm", _t(w), _t(b), _t(x), ctypes.c_float(eps), keep=(w, b, x))


def l2_norm(x, eps):
    return _mk("wrk_op_l2_norm", _t(x), ctypes.c_float(eps), keep=(x,))


def token_shift(cursors, time_mix, state, input, output, reversed):
    (pt, kt), (ps, ks) = _v(time_mix), _v(state)
    return _mk("wrk_op_token_shift", _t(cursors), pt, ps, _t(input), _t(output), int(reversed),
               keep=(cursors, kt, ks, input, output))


def channel_mix(cursors, state, r, v, x):
    ps, ks = _v(state)
    return _mk("wrk_op_channel_mix", _t(cursors), ps, _t(r), _t(v), _t(x), keep=(cursors, ks, r, v, x))


def channel_mix_v7(cursors, state, v, x):
    ps, ks = _v(state)
    return _mk("wrk_op_channel_mix_v7", _t(cursors), ps, _t(v), _t(x), keep=(cursors, ks, v, x))


def add_activate(input, output, act_x=ACT_NONE, act_y=ACT_NONE, act_out=ACT_NONE):
    (pi, ki), (po, ko) = _v(input), _v(output)
    return _mk("wrk_op_add_activate", pi, po, act_x, act_y, act_out, keep=(ki, ko))


def add(input, output):
    return add_activate(input, output)


def mul_activate(input, output, act_x=ACT_NONE, act_y=ACT_NONE, act_out=ACT_NONE):
    (pi, ki), (po, ko) = _v(input), _v(output)
    return _mk("wrk_op_mul_activate", pi, po, act_x, act_y, act_out, keep=(ki, ko))


def mul(input, output):
    return mul_activate(input, output)


def activate(x, act):
    px, kx = _v(x)
    return _mk("wrk_op_activate", px, act, keep=(kx,))


def blit(input, output):
    (pi, ki), (po, ko) = _v(input), _v(output)
    return _mk("wrk_op_blit", pi, po, keep=(ki, ko))


def broadcast(input, output):
    (pi, ki), (po, ko) = _v(input), _v(output)
    return _mk("wrk_op_broadcast", pi, po, keep=(ki, ko))


def blend(factor, input, output):
    return _mk("wrk_op_blend", _t(factor), _t(input), _t(output), keep=(factor, input, output))


def blend_lora(factor, xa, xb, output):
    (pa, ka), (pb, kb), (po, ko) = _v(xa), _v(xb), _v(output)
    return _mk("wrk_op_blend_lora", _t(factor), pa, pb, po, keep=(factor, ka, kb, ko))


def transpose(input, output):
    (pi, ki), (po, ko) = _v(input), _v(output)
    return _mk("wrk_op_transpose", pi, po, keep=(ki, ko))


def lerp(input, output, factor, reversed):
    (pi, ki), (po, ko), (pf, kf) = _v(input), _v(output), _v(factor)
    return _mk("wrk_op_lerp", pi, po, pf, int(reversed), keep=(ki, ko, kf))


def affine(x, scale, bias):
    return _mk("wrk_op_affine", _t(x), ctypes.c_float(scale), ctypes.c_float(bias), keep=(x,))


def control_k_v7(p, a, k):
    (pa, ka), (pk, kk) = _v(a), _v(k)
    return _mk("wrk_op_control_k_v7", _t(p), pa, pk, keep=(p, ka, kk))


def layer_norm_copy(w, b, delta, src, dst, eps):
    """dst <- layer_norm(src), after src <- src + delta when delta is not None: blit + layer_norm (+ add) in one launch."""
    return _mk("wrk_op_layer_norm_copy", _t(w), _t(b), _t(delta) if delta is not None else None, _t(src), _t(dst),
               ctypes.c_float(eps), keep=(w, b, delta, src, dst))


def token_shift_multi(cursors, state, input, time_mixes, outputs, reversed):
    """Up to six token shifts of one f16 input in one launch."""
    ps, ks = _v(state)
    n = len(time_mixes)
    mixes = (ctypes.c_void_p * n)(*[_t(t) for t in time_mixes])
    outs = (ctypes.c_void_p * n)(*[_t(t) for t in outputs])
    return _mk("wrk_op_token_shift_multi", _t(cursors), ps, _t(input), ctypes.c_uint32(n), mixes, outs, int(reversed),
               keep=(cursors, ks, input, *time_mixes, *outputs))


def pack_v7(k_k, k_a, k, v, a, kk, n, eps):
    """kk <- l2_norm(k * k_k), k <- control_k(k_a, a, k), n <- (k, v, a, kk) on f16 [S, H, T] tensors in one launch."""
    return _mk("wrk_op_pack_v7", _t(k_k), _t(k_a), _t(k), _t(v), _t(a), _t(kk), _t(n), ctypes.c_float(eps),
               keep=(k_k, k_a, k, v, a, kk, n))


def time_mix_blocks(per_token_decay, cursors, time_decay, time_first, state, k, v, r, x):
    """time_mix_v5 / time_mix_v6 computed in blocks of 16 tokens (heads of 64 channels)."""
    ps, ks = _v(state)
    return _mk("wrk_op_time_mix_blocks", int(per_token_decay), _t(cursors), _t(time_decay), _t(time_first), ps, _t(k), _t(v), _t(r),
               _t(x), keep=(cursors, time_decay, time_first, ks, k, v, r, x))


def token_shift_lora(cursors, time_mix, bias, state, input, output, reversed):
    """token_shift with factors f16(time_mix + bias): the add of the static factors and the shift in one launch."""
    (pt, kt), (pb, kb), (ps, ks) = _v(time_mix), _v(bias), _v(state)
    return _mk("wrk_op_token_shift_lora", _t(cursors), pt, pb, ps, _t(input), _t(output), int(reversed),
               keep=(cursors, kt, kb, ks, input, output))


def group_norm_gate(w, b, x, gate, output, eps, gate_act):
    """output <- act(gate) * f16(group_norm(x)): group norm + copy + gate in one launch; x is left as it was."""
    return _mk("wrk_op_group_norm_gate", _t(w), _t(b), _t(x), _t(gate), _t(output), ctypes.c_float(eps), int(gate_act),
               keep=(w, b, x, gate, output))


def channel_mix_add(cursors, state, r, v, x, residual, v7=False):
    """channel_mix (or channel_mix_v7) and the add of its result to the residual stream in one launch."""
    ps, ks = _v(state)
    return _mk("wrk_op_channel_mix_add", _t(cursors), ps, _t(r) if r is not None else None, _t(v), _t(x), _t(residual), int(v7),
               keep=(cursors, ks, r, v, x, residual))


def nf4_table():
    t = (ctypes.c_float * 16)()
    check(lib().wrk_nf4_table(t))
    return np.array(list(t), dtype=np.float32)


def sf4_table(nu=5.0):
    t = (ctypes.c_float * 16)()
    check(lib().wrk_sf4_table(ctypes.c_double(nu), t))
    return np.array(list(t), dtype=np.float32)


class Matrix:
    """`Matrix` of src/tensor/matrix.rs: Fp16 / Int8 {w, m} / Fp4 {q, w, m}."""

    def __init__(self, ctx, handle):
        self.ctx, self.handle = ctx, handle

    def __del__(self):
        if self.handle and _lib is not None:
            _lib.wrk_matrix_release(self.handle)
            self.handle = None

    @staticmethod
    def fp16(tensor):
        h = ctypes.c_void_p()
        check(lib().wrk_matrix_fp16(tensor.handle, ctypes.byref(h)))
        return Matrix(tensor.ctx, h)

    @staticmethod
    def quant_u8(tensor):
        h = ctypes.c_void_p()
        check(lib().wrk_matrix_quant_u8(tensor.handle, ctypes.byref(h)))
        return Matrix(tensor.ctx, h)

    @staticmethod
    def quant_nf4(tensor):
        h = ctypes.c_void_p()
        check(lib().wrk_matrix_quant_nf4(tensor.handle, ctypes.byref(h)))
        return Matrix(tensor.ctx, h)

    @staticmethod
    def quant_sf4(tensor, nu=5.0):
        h = ctypes.c_void_p()
        check(lib().wrk_matrix_quant_sf4(tensor.handle, ctypes.c_double(nu), ctypes.byref(h)))
        return Matrix(tensor.ctx, h)

    def parts(self):
        kind = ctypes.c_int32()
        w, m, q = ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_void_p()
        check(lib().wrk_matrix_parts(self.handle, ctypes.byref(kind), ctypes.byref(w), ctypes.byref(m),
                                     ctypes.byref(q)))
        out = []
        for h in (w, m, q):
            if h:
                check(lib().wrk_tensor_retain(h))
                out.append(Tensor(self.ctx, ctypes.c_void_p(h.value)))
            else:
                out.append(None)
        return kind.value, out[0], out[1], out[2]

    def matmul_op(self, input, output, act=ACT_NONE, turbo=False, sparse=False):
        (pi, ki), (po, ko) = _v(input), _v(output)
        fn = "wrk_matrix_matmul_op_sparse" if sparse else "wrk_matrix_matmul_op"
        return _mk(fn, self.handle, pi, po, act, int(turbo), keep=(self, ki, ko))


def matmul_group_op(matrices, inputs, outputs, acts=None, turbo=True):
    """Up to four `Matrix.matmul_op` of one point of a layer as one op (one tensor-core launch where the shapes allow)."""
    n = len(matrices)
    acts = list(acts) if acts is not None else [ACT_NONE] * n
    views = [x.as_view() if isinstance(x, Tensor) else x for x in list(inputs) + list(outputs)]
    ins = (CView * n)(*[v.c for v in views[:n]])
    outs = (CView * n)(*[v.c for v in views[n:]])
    ms = (ctypes.c_void_p * n)(*[m.handle for m in matrices])
    return _mk("wrk_matrix_matmul_group_op", ms, ins, outs, (ctypes.c_int32 * n)(*acts), ctypes.c_uint32(n), int(turbo),
               keep=(tuple(matrices), tuple(views)))


def gemv_int8_static(ctx, matrix, minmax, x, y, act=ACT_NONE, num_ctas=0, device=None):
    """`wrk_gemv_int8_static` (no counterpart in the reference): y[t][m] = act(W[m][:] . x[t][:]) on the context's
    stream without any allocation; the kernel's row-range table sits in a static device array (512 CTAs at most).
    `matrix` u8 [k, m], `minmax` f16 pairs, `x` f16 [k, t], `y` f32 [m, t]."""
    ptrs = []
    for t in (matrix, minmax, x, y):
        p = ctypes.c_void_p()
        check(lib().wrk_tensor_device_ptr(t.handle, ctypes.byref(p)))
        ptrs.append(p)
    stream = ctypes.c_void_p()
    check(lib().wrk_context_stream(ctx.handle, ctypes.byref(stream)))
    k, m = matrix.shape[0], matrix.shape[1]
    t = x.shape[1]
    if device is None:  # the context's own device
        dev = ctypes.c_int32()
        check(lib().wrk_context_device(ctx.handle, ctypes.byref(dev)))
        device = dev.value
    check(lib().wrk_gemv_int8_static(ctypes.c_int32(device), stream, ptrs[0], ptrs[1], ptrs[2], ptrs[3],
                                     ctypes.c_uint32(k), ctypes.c_uint32(m), ctypes.c_uint32(t), ctypes.c_int32(act),
                                     ctypes.c_uint32(num_ctas)))
