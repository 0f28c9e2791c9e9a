"""Supporting ops of the v5/v6/v7 jobs against the CPU oracle (layer/group norm, l2 norm, token
shift, channel mix, add/mul with activations, activate, blit, transpose, lerp, affine, control_k)."""
import numpy as np
import pytest

from oracle import oracle
from tests.util import assert_close, is_approx_eps

pytestmark = pytest.mark.gpu

DT = {np.float16: 1, np.float32: 0}


def _wdt(wrk, dt):
    return wrk.F16 if dt == np.float16 else wrk.F32


@pytest.mark.parametrize("dtype", [np.float16, np.float32])
@pytest.mark.parametrize("C,T", [(768, 5), (2048, 1), (64, 3)])
def test_layer_norm(wrk, ctx, dtype, C, T):
    rng = np.random.default_rng(C + T)
    x = (rng.standard_normal((T, C)) * 3 + 1).astype(dtype)
    w = (1 + rng.standard_normal(C) * 0.02).astype(np.float16)
    b = (rng.standard_normal(C) * 0.02).astype(np.float16)
    t_x = ctx.from_numpy(x)
    ctx.run(wrk.layer_norm(ctx.from_numpy(w), ctx.from_numpy(b), t_x, 1e-5))
    ref = x.copy()
    oracle.layer_norm(w, b, ref, 1e-5)
    assert_close(t_x.numpy().reshape(T, C), ref, "layer_norm")


@pytest.mark.parametrize("dtype", [np.float16, np.float32])
def test_group_norm(wrk, ctx, dtype):
    rng = np.random.default_rng(1)
    S, H, T = 64, 12, 7
    x = (rng.standard_normal((T, H, S)) * 2).astype(dtype)
    w = (1 + rng.standard_normal((H, S)) * 0.1).astype(np.float16)
    b = (rng.standard_normal((H, S)) * 0.1).astype(np.float16)
    t_x = ctx.from_numpy(x)
    ctx.run(wrk.group_norm(ctx.from_numpy(w), ctx.from_numpy(b), t_x, 64e-5))
    ref = x.copy()
    oracle.group_norm(w, b, ref, 64e-5, H)
    assert_close(t_x.numpy().reshape(T, H, S), ref, "group_norm")


@pytest.mark.parametrize("dt", [np.float32, np.float16])
def test_softmax_reference_test_shape(wrk, ctx, dt):
    # C, T, B of test_softmax (src/tensor/ops.rs:2632-2669): uniform(-5, 5) data, dense answer in f32
    rng = np.random.default_rng(42)
    x = (10.0 * (rng.random((2, 3, 1000), dtype=np.float32) - 0.5)).astype(dt)
    t_x = ctx.from_numpy(x)
    ctx.run(wrk.softmax(t_x))
    got = t_x.numpy().reshape(x.shape).astype(np.float32)
    ref = x.copy()
    oracle.softmax(ref)
    xf = x.astype(np.float32)  # the answer from the values the tensor holds (fp16-rounded in the fp16 case)
    e = np.exp(xf - xf.max(axis=-1, keepdims=True))
    dense = e / e.sum(axis=-1, keepdims=True)
    assert is_approx_eps(got, dense, 1e-3 if dt == np.float16 else 1e-4).all()
    assert_close(got, ref.astype(np.float32), "softmax vs oracle")
    assert np.allclose(got.sum(axis=-1), 1.0, atol=2e-3 if dt == np.float16 else 1e-5)


def test_softmax_vocabulary_row(wrk, ctx):
    # one row of 65536 logits with a wide range: the maximum is subtracted first
    rng = np.random.default_rng(7)
    x = (rng.standard_normal((1, 65536)) * 8.0 + 50.0).astype(np.float32)
    t_x = ctx.from_numpy(x)
    ctx.run(wrk.softmax(t_x))
    got = t_x.numpy().reshape(x.shape)
    ref = x.copy()
    oracle.softmax(ref)
    assert np.isfinite(got).all() and abs(float(got.sum()) - 1.0) < 1e-4
    assert np.allclose(got, ref, rtol=1e-4, atol=1e-9)
    assert int(got.argmax()) == int(x.argmax())


def test_l2_norm(wrk, ctx):
    rng = np.random.default_rng(2)
    x = rng.standard_normal((5, 8, 64)).astype(np.float16)
    t_x = ctx.from_numpy(x)
    ctx.run(wrk.l2_norm(t_x, 1e-12))
    ref = x.copy()
    oracle.l2_norm(ref, 1e-12)
    assert_close(t_x.numpy().reshape(x.shape), ref, "l2_norm")


@pytest.mark.parametrize("dtype", [np.float16, np.float32])
def test_recenter_and_rms_norm(wrk, ctx, dtype):
    rng = np.random.default_rng(21)
    C, T, B = 768, 5, 2
    x = (rng.standard_normal((B, T, C)) + 0.5).astype(dtype)
    w = (1 + 0.02 * rng.standard_normal(C)).astype(np.float16)
    b = (0.02 * rng.standard_normal(C)).astype(np.float16)
    t_x = ctx.from_numpy(x)
    ctx.run(wrk.recenter(t_x))
    ref = x.copy()
    oracle.recenter(ref)
    assert_close(t_x.numpy().reshape(x.shape), ref, "recenter")
    t_y = ctx.from_numpy(x)
    ctx.run(wrk.rms_norm(ctx.from_numpy(w), ctx.from_numpy(b), t_y, 1e-5))
    ref = x.copy()
    oracle.rms_norm(w, b, ref, 1e-5)
    assert_close(t_y.numpy().reshape(x.shape), ref, "rms_norm")
    with pytest.raises(wrk.WrkError) as e:
        wrk.rms_norm(ctx.from_numpy(w[:-4]), ctx.from_numpy(b), t_y, 1e-5)
    assert e.value.status == -5


@pytest.mark.parametrize("dtype", [np.float16, np.float32])
def test_embed_gather(wrk, ctx, dtype):
    # the device-side embedding gather: bit-exact rows of the fp16 matrix (widened exactly for f32 outputs)
    rng = np.random.default_rng(22)
    C, V, T, B = 512, 1000, 7, 3
    emb = rng.standard_normal((V, C)).astype(np.float16)
    tokens = rng.integers(0, V, (B, T)).astype(np.uint32)
    t_out = ctx.tensor(wrk.F16 if dtype == np.float16 else wrk.F32, [C, T, B])
    ctx.run(wrk.embed(ctx.from_numpy(tokens), ctx.from_numpy(emb), t_out))
    ref = np.zeros((B, T, C), dtype=dtype)
    oracle.embed(tokens, emb, ref)
    assert np.array_equal(t_out.numpy().reshape(ref.shape), ref)
    assert np.array_equal(ref, emb[tokens].astype(dtype))
    with pytest.raises(wrk.WrkError) as e:
        wrk.embed(ctx.from_numpy(tokens[:, :-1].copy()), ctx.from_numpy(emb), t_out)
    assert e.value.status == -5


def test_broadcast_and_blend(wrk, ctx):
    rng = np.random.default_rng(23)
    C, T, B = 128, 6, 4
    src = rng.standard_normal((2, 3, C)).astype(np.float16)
    t_dst = ctx.tensor(wrk.F32, [C, T, B], zeros=True)
    ctx.run(wrk.broadcast(ctx.from_numpy(src), t_dst))
    ref = np.zeros((B, T, C), dtype=np.float32)
    oracle.broadcast(src, ref)
    assert np.array_equal(t_dst.numpy().reshape(ref.shape), ref)
    assert np.array_equal(ref[3, 4], src[1, 1].astype(np.float32))
    # blend: output = f0 * input + f1 * output
    factor = np.array([0.25, 0.75, 0, 0], dtype=np.float32)
    a = rng.standard_normal((B, T, C)).astype(np.float16)
    o = rng.standard_normal((B, T, C)).astype(np.float16)
    t_o = ctx.from_numpy(o)
    ctx.run(wrk.blend(ctx.from_numpy(factor), ctx.from_numpy(a), t_o))
    ref = o.copy()
    oracle.blend(factor, a, ref)
    assert_close(t_o.numpy().reshape(ref.shape), ref, "blend")


def test_blend_lora(wrk, ctx):
    # LoRA merge W += alpha * B A on an fp16 matrix [K = 256 inputs, M = 192 rows]: xa [R, K], xb [R, M]
    rng = np.random.default_rng(24)
    R, K, M = 16, 256, 192
    xa = (0.1 * rng.standard_normal((K, R))).astype(np.float16)
    xb = (0.1 * rng.standard_normal((M, R))).astype(np.float16)
    w = (0.02 * rng.standard_normal((M, K))).astype(np.float16)
    factor = np.array([0.5, 1.0, 0, 0], dtype=np.float32)
    t_w = ctx.from_numpy(w)
    ctx.run(wrk.blend_lora(ctx.from_numpy(factor), ctx.from_numpy(xa), ctx.from_numpy(xb), t_w))
    ref = w.copy()
    oracle.blend_lora(factor, xa, xb, ref)
    assert_close(t_w.numpy().reshape(ref.shape), ref, "blend_lora", max_abs=2e-3)
    dense = 0.5 * xb.astype(np.float64) @ xa.astype(np.float64).T + w.astype(np.float64)
    assert np.max(np.abs(ref.astype(np.float64) - dense)) < 1e-3
    with pytest.raises(wrk.WrkError) as e:
        wrk.blend_lora(ctx.from_numpy(factor), ctx.from_numpy(xa[:-1].copy()), ctx.from_numpy(xb), t_w)
    assert e.value.status == -5


@pytest.mark.parametrize("reversed_", [True, False])
@pytest.mark.parametrize("per_token", [True, False])
def test_token_shift(wrk, ctx, reversed_, per_token):
    rng = np.random.default_rng(3)
    C, B, count = 256, 3, 5 if per_token else 1
    cursors = oracle.pack_cursors([(0, 0, 4), (2, 4, 1), (1, 5, 6)])
    T = 11
    state = rng.standard_normal((B, 66, C)).astype(np.float32)
    x = rng.standard_normal((T, C)).astype(np.float16)
    tm = rng.uniform(0, 1, (count, T if per_token else 1, C)).astype(np.float16)
    out = np.zeros((count, T, C), dtype=np.float16)
    t_state, t_out = ctx.from_numpy(state), ctx.tensor(wrk.F16, [C, T, count])
    ctx.run(wrk.token_shift(ctx.from_numpy(cursors), ctx.from_numpy(tm), t_state.view(y=(0, 65)), ctx.from_numpy(x),
                            t_out, reversed_))
    oracle.token_shift(cursors, tm, oracle.View(state, y=(0, 65)), x, out, reversed_)
    assert_close(t_out.numpy().reshape(out.shape), out, "token_shift")


@pytest.mark.parametrize("v7", [False, True])
def test_channel_mix(wrk, ctx, v7):
    rng = np.random.default_rng(4)
    C, B, T = 256, 3, 11
    cursors = oracle.pack_cursors([(0, 0, 4), (2, 4, 1), (1, 5, 6)])
    state = rng.standard_normal((B, 66, C)).astype(np.float32)
    r = rng.standard_normal((T, C)).astype(np.float16)
    v = rng.standard_normal((T, C)).astype(np.float16)
    x = rng.standard_normal((T, C)).astype(np.float16)
    t_state, t_x = ctx.from_numpy(state), ctx.from_numpy(x)
    if v7:
        op = wrk.channel_mix_v7(ctx.from_numpy(cursors), t_state.view(y=65), ctx.from_numpy(v), t_x)
    else:
        op = wrk.channel_mix(ctx.from_numpy(cursors), t_state.view(y=65), ctx.from_numpy(r), ctx.from_numpy(v), t_x)
    ctx.run(op)
    ref_x, ref_state = x.copy(), state.copy()
    oracle.channel_mix(cursors, oracle.View(ref_state, y=65), None if v7 else r, v, ref_x, v7=v7)
    assert_close(t_x.numpy().reshape(T, C), ref_x, "x")
    assert np.array_equal(t_state.numpy().reshape(state.shape), ref_state)


def test_binary_broadcast_and_activations(wrk, ctx):
    rng = np.random.default_rng(5)
    C, T, B = 128, 6, 5
    out0 = rng.standard_normal((B, T, C)).astype(np.float16)
    for shape in [(B, T, C), (B, 1, C), (1, 1, C)]:
        for is_mul, acts in [(False, (0, 0, 6)), (True, (7, 0, 0)), (False, (0, 0, 0)), (True, (0, 1, 2))]:
            inp = rng.standard_normal(shape).astype(np.float32)
            t_out = ctx.from_numpy(out0)
            fn = wrk.mul_activate if is_mul else wrk.add_activate
            ctx.run(fn(ctx.from_numpy(inp), t_out, *acts))
            ref = out0.copy()
            oracle.binary(is_mul, inp, ref, *acts)
            assert_close(t_out.numpy().reshape(ref.shape), ref, f"binary {shape} {is_mul} {acts}")


@pytest.mark.parametrize("act", range(8))
def test_activate(wrk, ctx, act):
    rng = np.random.default_rng(act)
    x = rng.standard_normal((3, 4, 64)).astype(np.float32)
    t_x = ctx.from_numpy(x)
    ctx.run(wrk.activate(t_x, act))
    ref = x.copy()
    oracle.activate(ref, act)
    assert_close(t_x.numpy().reshape(x.shape), ref, f"act {act}", max_abs=1e-4)


def test_blit_views_and_transpose(wrk, ctx):
    rng = np.random.default_rng(6)
    src = rng.standard_normal((4, 7, 64)).astype(np.float16)
    t_dst = ctx.tensor(wrk.F32, [64, 3, 9], zeros=True)
    ctx.run(wrk.blit(ctx.from_numpy(src).view(y=(2, 5), z=1), t_dst.view(z=4)))
    ref = np.zeros((9, 3, 64), dtype=np.float32)
    oracle.blit(oracle.View(src, y=(2, 5), z=1), oracle.View(ref, z=4))
    assert np.array_equal(t_dst.numpy().reshape(ref.shape), ref)
    t_tr = ctx.tensor(wrk.F16, [64, 4, 7])
    ctx.run(wrk.transpose(ctx.from_numpy(src), t_tr))
    assert np.array_equal(t_tr.numpy().reshape(7, 4, 64), src.transpose(1, 0, 2))
    with pytest.raises(wrk.WrkError) as e:
        wrk.blit(ctx.from_numpy(src), t_dst)
    assert e.value.status == -5


@pytest.mark.parametrize("reversed_", [True, False])
def test_lerp_affine_control_k(wrk, ctx, reversed_):
    rng = np.random.default_rng(7)
    T, C = 5, 128
    a = rng.standard_normal((T, C)).astype(np.float16)
    b = rng.standard_normal((T, C)).astype(np.float16)
    f = rng.uniform(0, 1, (T, C)).astype(np.float16)
    t_b = ctx.from_numpy(b)
    ctx.run(wrk.lerp(ctx.from_numpy(a), t_b, ctx.from_numpy(f), reversed_))
    ref = b.copy()
    oracle.lerp(a, ref, f, reversed_)
    assert_close(t_b.numpy().reshape(T, C), ref, "lerp")
    ctx.run(wrk.affine(t_b, 0.5, 0.0))
    oracle.affine(ref, 0.5, 0.0)
    assert_close(t_b.numpy().reshape(T, C), ref, "affine")
    p = rng.uniform(0, 1, C).astype(np.float16)
    ctx.run(wrk.control_k_v7(ctx.from_numpy(p), ctx.from_numpy(f), t_b))
    oracle.control_k_v7(p, f, ref)
    assert_close(t_b.numpy().reshape(T, C), ref, "control_k")


def test_op_list_encode_and_graph(wrk, ctx):
    # deferred ops: nothing runs at build time; a list runs in order; a graph replays the same work
    x = np.ones((2, 64), dtype=np.float32)
    t_x = ctx.from_numpy(x)
    ops = wrk.op_list([wrk.affine(t_x, 2.0, 1.0), wrk.affine(t_x, 3.0, 0.0)])
    assert ops.num_atoms() == 2
    assert np.array_equal(t_x.numpy().reshape(x.shape), x)
    cmd = ctx.encode(ops, use_graph=True)
    before = ctx.launch_count()
    cmd.submit()
    assert np.array_equal(t_x.numpy().reshape(x.shape), (x * 2 + 1) * 3)
    cmd.submit()
    assert np.array_equal(t_x.numpy().reshape(x.shape), (((x * 2 + 1) * 3) * 2 + 1) * 3)
    assert ctx.launch_count() - before == 4
    assert ctx.device_status() == 0


# ---- merged elementwise launches: bit-identical to the runs of single ops they stand for ----------------

@pytest.mark.parametrize("reversed_", [False, True])
@pytest.mark.parametrize("count", [1, 2, 6])
def test_token_shift_multi_equals_the_single_shifts(wrk, ctx, reversed_, count):
    rng = np.random.default_rng(31)
    C, B, T = 256, 3, 11
    cursors = ctx.from_numpy(oracle.pack_cursors([(0, 0, 4), (2, 4, 1), (1, 5, 6)]))
    state = ctx.from_numpy(rng.standard_normal((B, 66, C)).astype(np.float32))
    x = ctx.from_numpy(rng.standard_normal((T, C)).astype(np.float16))
    mixes = [ctx.from_numpy(rng.uniform(0, 1, (C,)).astype(np.float16)) for _ in range(count)]
    single = [ctx.tensor(wrk.F16, [C, T, 1]) for _ in range(count)]
    multi = [ctx.tensor(wrk.F16, [C, T, 1]) for _ in range(count)]
    for m, o in zip(mixes, single):
        ctx.run(wrk.token_shift(cursors, m, state.view(y=(0, 1)), x, o, reversed_))
    ctx.run(wrk.token_shift_multi(cursors, state.view(y=(0, 1)), x, mixes, multi, reversed_))
    for a, b in zip(single, multi):
        assert np.array_equal(a.numpy(), b.numpy())
    with pytest.raises(wrk.WrkError):
        wrk.token_shift_multi(cursors, state.view(y=(0, 1)), x, mixes * 7, multi * 7, reversed_)


@pytest.mark.parametrize("C,T", [(256, 9), (4096, 5), (12288, 3)])  # one warp per row / rows kept in registers / three passes
@pytest.mark.parametrize("with_delta", [False, True])
def test_layer_norm_copy_equals_add_blit_layer_norm(wrk, ctx, C, T, with_delta):
    rng = np.random.default_rng(32)
    w = ctx.from_numpy(rng.standard_normal(C).astype(np.float16))
    b = ctx.from_numpy(rng.standard_normal(C).astype(np.float16))
    x0 = rng.standard_normal((T, C)).astype(np.float16)
    d0 = rng.standard_normal((T, C)).astype(np.float16)
    x_a, x_b, delta = ctx.from_numpy(x0), ctx.from_numpy(x0), ctx.from_numpy(d0)
    out_a, out_b = ctx.tensor(wrk.F16, [C, T, 1]), ctx.tensor(wrk.F16, [C, T, 1])
    if with_delta:
        ctx.run(wrk.add(delta, x_a))
    ctx.run(wrk.blit(x_a, out_a))
    ctx.run(wrk.layer_norm(w, b, out_a, 1e-5))
    ctx.run(wrk.layer_norm_copy(w, b, delta if with_delta else None, x_b, out_b, 1e-5))
    assert np.array_equal(x_a.numpy(), x_b.numpy())
    assert np.array_equal(out_a.numpy(), out_b.numpy())
    if with_delta:
        with pytest.raises(wrk.WrkError):
            wrk.layer_norm_copy(w, b, x_b, x_b, out_b, 1e-5)


def test_pack_v7_equals_the_eight_ops(wrk, ctx):
    rng = np.random.default_rng(33)
    S, H, T = 64, 6, 7
    C = S * H
    k0 = rng.standard_normal((T, C)).astype(np.float16)
    v0 = rng.standard_normal((T, C)).astype(np.float16)
    a0 = rng.uniform(0, 1, (T, C)).astype(np.float16)
    k_k = ctx.from_numpy(rng.uniform(0.5, 1.5, C).astype(np.float16))
    k_a = ctx.from_numpy(rng.uniform(0.5, 1.5, C).astype(np.float16))
    # the reference's op list (src/runtime/v7.rs:888-891, 925-928)
    k, v, a = ctx.from_numpy(k0), ctx.from_numpy(v0), ctx.from_numpy(a0)
    kk, n = ctx.tensor(wrk.F16, [C, T, 1]), ctx.tensor(wrk.F16, [C, T, 4])
    ctx.run(wrk.blit(k, kk))
    ctx.run(wrk.mul(k_k, kk))
    ctx.run(wrk.l2_norm(kk.reshape(S, H, T), 1e-12))
    ctx.run(wrk.control_k_v7(k_a, a, k))
    for z, t in enumerate((k, v, a, kk)):
        ctx.run(wrk.blit(t, n.view(z=z)))
    # one launch
    k2, v2, a2 = ctx.from_numpy(k0), ctx.from_numpy(v0), ctx.from_numpy(a0)
    kk2, n2 = ctx.tensor(wrk.F16, [S, H, T]), ctx.tensor(wrk.F16, [S, H, T, 4])
    ctx.run(wrk.pack_v7(k_k, k_a, k2.reshape(S, H, T), v2.reshape(S, H, T), a2.reshape(S, H, T), kk2, n2, 1e-12))
    assert np.array_equal(k.numpy().ravel(), k2.numpy().ravel())
    assert np.array_equal(kk.numpy().ravel(), kk2.numpy().ravel())
    assert np.array_equal(n.numpy().ravel(), n2.numpy().ravel())
    assert float(np.abs(kk2.numpy()).max()) > 0


def test_token_shift_lora_equals_add_then_shift(wrk, ctx):
    rng = np.random.default_rng(34)
    C, B, T, Z = 256, 3, 11, 5
    cursors = ctx.from_numpy(oracle.pack_cursors([(0, 0, 4), (2, 4, 1), (1, 5, 6)]))
    state = ctx.from_numpy(rng.standard_normal((B, 66, C)).astype(np.float32))
    x = ctx.from_numpy(rng.standard_normal((T, C)).astype(np.float16))
    lora0 = rng.uniform(-0.3, 0.3, (Z, T, C)).astype(np.float16)
    bias = ctx.from_numpy(rng.uniform(0.2, 0.8, (Z, 1, C)).astype(np.float16))
    lora_a, lora_b = ctx.from_numpy(lora0), ctx.from_numpy(lora0)
    out_a, out_b = ctx.tensor(wrk.F16, [C, T, Z]), ctx.tensor(wrk.F16, [C, T, Z])
    ctx.run(wrk.add(bias, lora_a))
    ctx.run(wrk.token_shift(cursors, lora_a, state.view(y=(0, 1)), x, out_a, True))
    ctx.run(wrk.token_shift_lora(cursors, lora_b, bias, state.view(y=(0, 1)), x, out_b, True))
    assert np.array_equal(out_a.numpy(), out_b.numpy())
    assert np.array_equal(lora_b.numpy().ravel(), lora0.ravel())  # the adapter's output is left alone
    want = np.zeros((Z, T, C), dtype=np.float16)
    oracle.token_shift(oracle.pack_cursors([(0, 0, 4), (2, 4, 1), (1, 5, 6)]), lora_a.numpy().reshape(Z, T, C),
                       oracle.View(state.numpy().reshape(B, 66, C), y=(0, 1)), x.numpy().reshape(T, C), want, True)
    assert_close(out_b.numpy().reshape(Z, T, C), want, "token_shift_lora")


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
def test_group_norm_gate_equals_norm_copy_gate(wrk, ctx, dtype):
    rng = np.random.default_rng(35)
    S, H, T = 64, 5, 9
    x0 = rng.standard_normal((T, H, S)).astype(dtype)
    w = ctx.from_numpy(rng.standard_normal((H, S)).astype(np.float16))
    b = ctx.from_numpy(rng.standard_normal((H, S)).astype(np.float16))
    gate = ctx.from_numpy(rng.standard_normal((T, H * S)).astype(np.float16))
    x_a, x_b = ctx.from_numpy(x0), ctx.from_numpy(x0)
    out_a, out_b = ctx.tensor(wrk.F16, [H * S, T, 1]), ctx.tensor(wrk.F16, [H * S, T, 1])
    ctx.run(wrk.group_norm(w, b, x_a, 64e-5))
    ctx.run(wrk.blit(x_a.reshape(H * S, T), out_a))
    ctx.run(wrk.mul_activate(gate, out_a, wrk.ACT_SILU, wrk.ACT_NONE, wrk.ACT_NONE))
    ctx.run(wrk.group_norm_gate(w, b, x_b, gate, out_b, 64e-5, wrk.ACT_SILU))
    assert np.array_equal(out_a.numpy(), out_b.numpy())
    assert np.array_equal(x_b.numpy().ravel(), x0.ravel())


@pytest.mark.parametrize("v7", [False, True])
def test_channel_mix_add_equals_mix_then_add(wrk, ctx, v7):
    rng = np.random.default_rng(36)
    C, B, T = 256, 3, 11
    cursors = ctx.from_numpy(oracle.pack_cursors([(0, 0, 4), (2, 4, 1), (1, 5, 6)]))
    state0 = rng.standard_normal((B, 66, C)).astype(np.float32)
    r = ctx.from_numpy(rng.standard_normal((T, C)).astype(np.float16))
    v = ctx.from_numpy(rng.standard_normal((T, C)).astype(np.float16))
    x0 = rng.standard_normal((T, C)).astype(np.float16)
    res0 = rng.standard_normal((T, C)).astype(np.float16)
    st_a, st_b = ctx.from_numpy(state0), ctx.from_numpy(state0)
    x_a, x_b, res_a, res_b = ctx.from_numpy(x0), ctx.from_numpy(x0), ctx.from_numpy(res0), ctx.from_numpy(res0)
    if v7:
        ctx.run(wrk.channel_mix_v7(cursors, st_a.view(y=65), v, x_a))
    else:
        ctx.run(wrk.channel_mix(cursors, st_a.view(y=65), r, v, x_a))
    ctx.run(wrk.add(x_a, res_a))
    ctx.run(wrk.channel_mix_add(cursors, st_b.view(y=65), None if v7 else r, v, x_b, res_b, v7))
    assert np.array_equal(x_a.numpy(), x_b.numpy())
    assert np.array_equal(res_a.numpy(), res_b.numpy())
    assert np.array_equal(st_a.numpy(), st_b.numpy())
