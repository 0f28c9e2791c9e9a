"""The CPU oracle against independent restatements and against the properties the reference's own
tests assert (src/tensor/ops.rs:2914-3257).  No GPU needed."""
import numpy as np
import pytest

from oracle import oracle
from tests.golden import reference_answers as ra
from tests.util import is_approx_eps


def _int8_numpy(m):
    """Independent vectorised restatement of quant_mat_int8.wgsl for whole blocks."""
    flat = m.reshape(-1, 128).astype(np.float32)
    mn, mx = flat.min(axis=1, keepdims=True), flat.max(axis=1, keepdims=True)
    with np.errstate(invalid="ignore", divide="ignore"):
        x = (flat - mn) / (mx - mn)
    x = np.where(x > 0, x, np.float32(0))
    x = np.minimum(x, np.float32(1))
    q = np.floor(np.float32(0.5) + np.float32(255) * x).astype(np.uint8)
    return q.reshape(m.shape), np.concatenate([mn, mx], axis=1).astype(np.float16).reshape(-1)


@pytest.mark.parametrize("c,r", [(2560, 2048), (320, 64)])
def test_int8_reference_test_properties(c, r):
    rng = np.random.default_rng(42)
    m = (10.0 * (rng.random((r, c), dtype=np.float32) - 0.5)).astype(np.float16)
    q, mm = oracle.quantize_mat_int8(m)
    q2, mm2 = _int8_numpy(m)
    assert np.array_equal(q, q2) and np.array_equal(mm.view(np.uint16), mm2.view(np.uint16))
    # the reference test's CPU answer: round((v - min) / (max - min) * 255), asserted within +-1
    flat = m.reshape(-1, 128).astype(np.float32)
    mn, mx = flat.min(axis=1, keepdims=True), flat.max(axis=1, keepdims=True)
    ans = np.round((flat - mn) / (mx - mn) * 255.0)
    assert (np.abs(ans - q.reshape(-1, 128).astype(np.float32)) < 2).all()
    assert is_approx_eps(mm.reshape(-1, 2)[:, 0], mn[:, 0], 0.01).all()
    assert is_approx_eps(mm.reshape(-1, 2)[:, 1], mx[:, 0], 0.01).all()


def test_int8_known_answers():
    m = np.zeros((1, 128), dtype=np.float16)
    m[0, :] = np.linspace(0, 1, 128).astype(np.float16)
    m[0, 0], m[0, 127] = 0.0, 1.0
    q, mm = oracle.quantize_mat_int8(m)
    assert q[0, 0] == 0 and q[0, 127] == 255
    assert mm[0] == 0.0 and mm[1] == 1.0
    v = m[0].astype(np.float32)
    assert np.array_equal(q[0], np.floor(np.float32(0.5) + np.float32(255) * v).astype(np.uint8))
    # degenerate and all-zero blocks quantize to 0
    q, mm = oracle.quantize_mat_int8(np.full((1, 128), 0.25, dtype=np.float16))
    assert (q == 0).all() and mm[0] == mm[1] == 0.25


@pytest.mark.parametrize("c,r", [(2560, 2048), (320, 64)])
def test_nf4_reference_test_properties(c, r):
    rng = np.random.default_rng(42)
    m = rng.standard_normal((r, c)).astype(np.float16)
    q, am = oracle.quantize_mat_nf4(m)
    flat = m.reshape(-1, 64).astype(np.float32)
    absmax = np.abs(flat).max(axis=1, keepdims=True)
    assert np.array_equal(am.view(np.uint16), absmax.astype(np.float16).reshape(-1).view(np.uint16))
    # the reference test's CPU answer: value / absmax, strict '<' first-wins arg-min; it asserts the
    # nibbles equal.  The shader (and the oracle) use value * (1 / absmax) with '<=': the two may
    # only differ where the value sits within rounding of a midpoint between two code-book entries.
    x = flat / absmax
    ans = np.abs(x[..., None] - oracle.NF4_TABLE[None, None, :]).argmin(axis=-1).astype(np.uint8)
    packed = q.reshape(-1, 32)
    nib = np.empty_like(ans)
    nib[:, 0::2], nib[:, 1::2] = packed & 15, packed >> 4
    diff = nib != ans
    assert diff.mean() < 1e-4
    mids = (oracle.NF4_TABLE[:-1] + oracle.NF4_TABLE[1:]) / 2
    if diff.any():
        assert np.abs(x[diff][:, None] - mids[None, :]).min(axis=1).max() < 1e-6
    # packing order: element 0 of every pair in the low nibble
    assert (nib[:, 0] == (packed[:, 0] & 15)).all()


def test_nf4_known_answers():
    m = np.zeros((1, 64), dtype=np.float16)
    m[0, :16] = oracle.NF4_TABLE.astype(np.float16)
    q, am = oracle.quantize_mat_nf4(m)
    assert am[0] == 1.0
    assert list(q[0, :8]) == [0x10, 0x32, 0x54, 0x76, 0x98, 0xBA, 0xDC, 0xFE]
    assert (q[0, 8:] == 0x77).all()  # zeros map to index 7 (0.0)
    q, am = oracle.quantize_mat_nf4(np.zeros((1, 64), dtype=np.float16))
    assert (q == 0).all() and am[0] == 0.0  # 0 * inf = NaN: no comparison succeeds → index 0


@pytest.mark.parametrize("kind", ["int8", "nf4", "fp16"])
def test_matmul_matches_dequant_dot(kind):
    rng = np.random.default_rng(1)
    K, M, N = 256, 24, 5
    w = (10.0 * (rng.random((M, K), dtype=np.float32) - 0.5)).astype(np.float16)
    x = (10.0 * (rng.random((N, K), dtype=np.float32) - 0.5)).astype(np.float16)
    if kind == "int8":
        q, s = oracle.quantize_mat_int8(w)
        deq, k = oracle.dequant_int8(q, s), oracle.MAT_INT8
    elif kind == "nf4":
        q, s = oracle.quantize_mat_nf4(w)
        deq, k = oracle.dequant_nf4(q, s), oracle.MAT_NF4
    else:
        q, s, deq, k = w, None, w.astype(np.float32), oracle.MAT_FP16
    ans = x.astype(np.float64) @ deq.astype(np.float64).T
    for mode in (0, 1):
        y = np.zeros((N, M), dtype=np.float32)
        oracle.matmul(k, q, s, x, y, mode=mode)
        assert is_approx_eps(y, ans, 0.01).all()
    y16 = np.zeros((N, M), dtype=np.float16)
    oracle.matmul(k, q, s, x, y16, act=oracle.ACT_SQUARED_RELU)
    assert is_approx_eps(y16, np.maximum(ans, 0) ** 2, 0.01).all()


def test_wkv6_against_dense_numpy():
    rng = np.random.default_rng(2)
    S, H, T = 64, 2, 5
    C = S * H
    k, v, r = (rng.standard_normal((T, H, S)).astype(np.float32) * 0.5 for _ in range(3))
    x = rng.standard_normal((T, H, S)).astype(np.float32)
    w = np.exp(-np.exp(rng.uniform(-6, 1, (T, H, S)))).astype(np.float32)
    u = rng.uniform(-1, 1, (H, S)).astype(np.float32)
    state = (rng.standard_normal((1, S + 2, C)) * 0.1).astype(np.float32)
    cursors = oracle.pack_cursors([(0, 0, T)])
    x_in, st = x.copy(), state.copy()
    oracle.time_mix_v56(True, cursors, w, u, oracle.View(st, y=(0, S + 1)), k, v, r, x, S, H)
    # dense restatement: per head S[i, j]
    Sm = state[0, 1:S + 1].reshape(S, H, S).transpose(1, 0, 2).astype(np.float64)  # [h, i, j]
    for t in range(T):
        for h in range(H):
            kv = np.outer(k[t, h], v[t, h])
            y = (r[t, h][:, None] * (u[h][:, None] * kv + Sm[h])).sum(axis=0)
            Sm[h] = w[t, h][:, None] * Sm[h] + kv
            assert np.allclose(x[t, h], y, atol=1e-4)
    assert np.allclose(st[0, 1:S + 1].reshape(S, H, S).transpose(1, 0, 2), Sm, atol=1e-4)
    assert np.array_equal(st[0, 0], x_in[T - 1].reshape(-1))  # token-shift carry = last input row
    assert np.array_equal(st[0, S + 1], state[0, S + 1])


def test_wkv7_against_dense_numpy():
    rng = np.random.default_rng(3)
    S, H, T = 64, 2, 4
    C = S * H
    r, wr, k, v = (rng.standard_normal((T, H, S)).astype(np.float32) for _ in range(4))
    a = rng.uniform(0, 1, (T, H, S)).astype(np.float32)
    kk = rng.standard_normal((T, H, S)).astype(np.float32)
    kk /= np.linalg.norm(kk, axis=-1, keepdims=True)
    n = np.stack([k, v, a, kk])
    x = rng.standard_normal((T, H, S)).astype(np.float32)
    state = (rng.standard_normal((1, S + 2, C)) * 0.1).astype(np.float32)
    st = state.copy()
    oracle.time_mix_v7(oracle.pack_cursors([(0, 0, T)], wide=True), oracle.View(st, y=(0, S + 1)), r, wr, n, x, S, H)
    Sm = state[0, 1:S + 1].reshape(S, H, S).transpose(1, 0, 2).astype(np.float64)
    for t in range(T):
        for h in range(H):
            w = np.exp(-0.606531 / (1 + np.exp(-wr[t, h].astype(np.float64))))
            sa = -(Sm[h] * kk[t, h][:, None]).sum(axis=0)
            Sm[h] = Sm[h] * w[:, None] + np.outer(k[t, h], v[t, h]) + np.outer(kk[t, h] * a[t, h], sa)
            y = (r[t, h][:, None] * Sm[h]).sum(axis=0)
            assert np.allclose(x[t, h], y, atol=1e-3)


def test_packed_cursor_wraps_like_the_reference():
    # Cursor::pack keeps 8 bits of batch and len and 16 of token (src/tensor/mod.rs:53-60)
    packed = oracle.pack_cursors([(3, 0, 256)])
    assert packed.shape == (256,) and packed[0] == 3  # len 256 wraps to 0
    packed = oracle.pack_cursors([(1, 5, 7), (2, 12, 0), (4, 12, 2)])
    assert list(packed) == [1 | 5 << 8 | 7 << 24] * 7 + [4 | 12 << 8 | 2 << 24] * 2


def test_softmax_against_dense_numpy():
    # the arithmetic of src/shaders/softmax.wgsl against a float64 restatement, on the reference test's shape
    rng = np.random.default_rng(42)
    x = (10.0 * (rng.random((2, 3, 1000), dtype=np.float32) - 0.5)).astype(np.float32)
    got = x.copy()
    oracle.softmax(got)
    x64 = x.astype(np.float64)
    e = np.exp(x64 - x64.max(axis=-1, keepdims=True))
    assert np.allclose(got, e / e.sum(axis=-1, keepdims=True), rtol=1e-5, atol=1e-9)
    h = x.astype(np.float16)  # fp16 tensors: fp16 inputs, f32 math, fp16 outputs
    h64 = h.astype(np.float64)
    oracle.softmax(h)
    eh = np.exp(h64 - h64.max(axis=-1, keepdims=True))
    assert np.allclose(h.astype(np.float64), eh / eh.sum(axis=-1, keepdims=True), rtol=2e-3, atol=1e-7)


def test_load_time_ops_against_dense_numpy():
    # recenter / rms_norm (normalize.wgsl), embed (embed.wgsl), broadcast (reshape.wgsl), blend, blend_lora
    rng = np.random.default_rng(9)
    x = (rng.standard_normal((2, 3, 256)) + 0.5).astype(np.float32)
    got = x.copy()
    oracle.recenter(got)
    assert np.allclose(got, x - x.mean(axis=-1, keepdims=True), atol=1e-5)
    w = (1 + 0.02 * rng.standard_normal(256)).astype(np.float16)
    b = (0.02 * rng.standard_normal(256)).astype(np.float16)
    got = x.copy()
    oracle.rms_norm(w, b, got, 1e-5)
    x64 = x.astype(np.float64)
    want = x64 / np.sqrt((x64 ** 2).mean(axis=-1, keepdims=True) + 1e-5) * w.astype(np.float64) + b.astype(np.float64)
    assert np.allclose(got, want, atol=1e-5)
    emb = rng.standard_normal((50, 64)).astype(np.float16)
    tokens = rng.integers(0, 50, (2, 5)).astype(np.uint32)
    out = np.zeros((2, 5, 64), dtype=np.float32)
    oracle.embed(tokens, emb, out)
    assert np.array_equal(out, emb[tokens].astype(np.float32))
    src = rng.standard_normal((2, 3, 64)).astype(np.float16)
    dst = np.zeros((4, 6, 64), dtype=np.float16)
    oracle.broadcast(src, dst)
    assert np.array_equal(dst, np.tile(src, (2, 2, 1)))
    a, o = rng.standard_normal((3, 64)).astype(np.float32), rng.standard_normal((3, 64)).astype(np.float32)
    want = np.float32(0.25) * a + np.float32(0.75) * o
    oracle.blend([0.25, 0.75, 0, 0], a, o)
    assert np.array_equal(o, want)
    xa = (0.1 * rng.standard_normal((32, 8))).astype(np.float16)
    xb = (0.1 * rng.standard_normal((24, 8))).astype(np.float16)
    m = (0.02 * rng.standard_normal((24, 32))).astype(np.float16)
    want = 2.0 * xb.astype(np.float64) @ xa.astype(np.float64).T + 0.5 * m.astype(np.float64)
    oracle.blend_lora([2.0, 0.5, 0, 0], xa, xb, m)
    assert np.allclose(m.astype(np.float64), want, atol=1e-3)


def test_wkv4_against_dense_numpy():
    # time_mix_v4.wgsl keeps (aa, bb, pp) = (numerator, denominator, running exponent) of
    # wkv_t = (sum_{s<t} e^{(t-1-s) w + k_s} v_s + e^{u + k_t} v_t) / (sum_{s<t} e^{(t-1-s) w + k_s} + e^{u + k_t});
    # the float64 restatement evaluates those sums directly (w <= 0 is the per-step log decay)
    rng = np.random.default_rng(4)
    C, T = 64, 9
    k, v, r = (rng.standard_normal((T, C)).astype(np.float32) for _ in range(3))
    x = rng.standard_normal((T, C)).astype(np.float32)
    w = (-np.exp(rng.uniform(-3, 0.5, C))).astype(np.float32)
    u = rng.uniform(-1, 1, C).astype(np.float32)
    state = np.zeros((2, 4, C), dtype=np.float32)
    state[:, 3] = -1e30  # the empty history: pp = -inf stand-in, aa = bb = 0
    cursors = oracle.pack_cursors([(1, 0, 6), (0, 6, 3)], wide=True)
    x_in, st = x.copy(), state.copy()
    oracle.time_mix_v4(cursors, w, u, st, k, v, r, x)
    for batch, t0, n in ((1, 0, 6), (0, 6, 3)):
        k64, v64 = k[t0:t0 + n].astype(np.float64), v[t0:t0 + n].astype(np.float64)
        for t in range(n):
            decay = np.array([(t - 1 - s_) * w.astype(np.float64) + k64[s_] for s_ in range(t)]).reshape(t, C)
            num = (np.exp(decay) * v64[:t]).sum(axis=0) + np.exp(u + k64[t]) * v64[t]
            den = np.exp(decay).sum(axis=0) + np.exp(u + k64[t])
            want = num / den / (1.0 + np.exp(-r[t0 + t].astype(np.float64)))
            assert np.allclose(x[t0 + t], want, rtol=1e-4, atol=1e-5), (batch, t)
        assert np.array_equal(st[batch, 0], x_in[t0 + n - 1])  # token-shift carry = the sequence's last input row
        # state after n tokens: aa / bb = decayed averages, in the shader's scaled form aa e^{pp}, bb e^{pp}
        decay = np.array([(n - 1 - s_) * w.astype(np.float64) + k64[s_] for s_ in range(n)])
        assert np.allclose(st[batch, 1] * np.exp(st[batch, 3].astype(np.float64)), (np.exp(decay) * v64).sum(axis=0), rtol=1e-4)
        assert np.allclose(st[batch, 2] * np.exp(st[batch, 3].astype(np.float64)), np.exp(decay).sum(axis=0), rtol=1e-4)


@pytest.mark.parametrize("c,r,t", [(2560, 2048, 8), (320, 64, 320)])
def test_int8_against_the_reference_tests_own_answer_code(c, r, t):
    # tests/golden/reference_answers.py restates the host code of test_matmul_int8; the oracle stands where the
    # shaders stand in that test and must pass the same three comparisons
    m, x = ra.int8_inputs(c, r, t)
    q_ans, mn, mx = ra.int8_quantize(m)
    q, mm = oracle.quantize_mat_int8(m)
    assert ra.is_approx_eps(mm.reshape(-1, 2)[:, 0], mn, 0.01).all() and ra.is_approx_eps(mm.reshape(-1, 2)[:, 1], mx, 0.01).all()
    assert (np.abs(q.astype(np.int32) - q_ans.astype(np.int32)) < 2).all()
    # the test feeds the *shader's* bytes to its answer loop
    ans = ra.int8_answer(q, mn, mx, x)
    for mode in (0, 1):
        if mode == 1 and c % 128:
            continue
        y = np.zeros((t, r), dtype=np.float32)
        oracle.matmul(oracle.MAT_INT8, q, mm, x, y, mode=mode)
        assert ra.is_approx_eps(y, ans, 0.01).all(), f"mode {mode}"


@pytest.mark.parametrize("c,r,t", [(2560, 2048, 8), (320, 64, 320)])
def test_nf4_against_the_reference_tests_own_answer_code(c, r, t):
    m, x = ra.nf4_inputs(c, r, t)
    idx, packed, absmax = ra.nf4_quantize(m)
    q, am = oracle.quantize_mat_nf4(m)
    assert ra.is_approx_eps(am, absmax, 0.01).all()
    assert np.array_equal(q.reshape(packed.shape), packed)  # the test asserts the packed nibbles equal
    ans = ra.nf4_answer(idx, absmax, x)
    for mode in (0, 1):
        y = np.zeros((t, r), dtype=np.float32)
        oracle.matmul(oracle.MAT_NF4, q, am, x, y, mode=mode)
        assert ra.is_approx_eps(y, ans, 0.01).all(), f"mode {mode}"
