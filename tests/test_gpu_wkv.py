"""WKV recurrences (time_mix_v5 / v6 / v7, time_first_v7) against the CPU oracle.

The reference has no test for these kernels: the oracle restates the shader text
(time_mix_v5.wgsl, time_mix_v6.wgsl, time_mix_v7.wgsl) and parity is otherwise unpinned.
Tolerance: max-abs 2e-2, cosine >= 0.9995 on outputs and on the recurrent state.
"""
import numpy as np
import pytest

from oracle import oracle
from tests.util import assert_close

pytestmark = pytest.mark.gpu

S = 64


def _cursors(seqs, wide):
    """seqs: list of (batch, len) in stack order → per-token cursors."""
    cur, tok = [], 0
    for b, n in seqs:
        cur.append((b, tok, n))
        tok += n
    return oracle.pack_cursors(cur, wide=wide), tok


def _v56_case(wrk, ctx, version, H, seqs, B, wide, dtype=np.float32, seed=0, S=S, blocks=False):
    rng = np.random.default_rng(seed)
    C = S * H
    cursors, T = _cursors(seqs, wide)
    k = (rng.standard_normal((T, H, S)) * 0.5).astype(dtype)
    v = (rng.standard_normal((T, H, S)) * 0.5).astype(dtype)
    r = (rng.standard_normal((T, H, S)) * 0.5).astype(dtype)
    x = rng.standard_normal((T, H, S)).astype(dtype)
    u = rng.uniform(-1, 1, (H, S)).astype(np.float32)
    if version == 6:
        w = np.exp(-np.exp(rng.uniform(-6, 1, (T, H, S)))).astype(np.float32)
    else:
        w = np.exp(-np.exp(rng.uniform(-6, 1, (H, S)))).astype(np.float32)
    state = (rng.standard_normal((B, S + 2, C)) * 0.1).astype(np.float32)

    t_state = ctx.from_numpy(state)
    t_x = ctx.from_numpy(x)
    fn = wrk.time_mix_v6 if version == 6 else wrk.time_mix_v5
    if blocks:
        fn = lambda *args: wrk.time_mix_blocks(version == 6, *args)
    op = fn(ctx.from_numpy(cursors), ctx.from_numpy(w), ctx.from_numpy(u), t_state.view(y=(0, S + 1)),
            ctx.from_numpy(k), ctx.from_numpy(v), ctx.from_numpy(r), t_x)
    ctx.run(op)
    got_x, got_state = t_x.numpy().reshape(T, H, S), t_state.numpy().reshape(B, S + 2, C)

    ref_x, ref_state = x.copy(), state.copy()
    oracle.time_mix_v56(version == 6, cursors, w, u, oracle.View(ref_state, y=(0, S + 1)), k, v, r, ref_x, S, H)
    return got_x, got_state, ref_x, ref_state


@pytest.mark.parametrize("version", [5, 6])
@pytest.mark.parametrize("wide", [False, True])
def test_v56_multi_sequence(wrk, ctx, version, wide):
    # four batch slots, slot 2 idle; runs of different lengths including a single token
    gx, gs, rx, rs = _v56_case(wrk, ctx, version, 4, [(0, 5), (1, 1), (3, 9)], 4, wide, seed=version)
    assert_close(gx, rx, "x")
    assert_close(gs, rs, "state")
    # the idle slot's state is untouched, the FFN carry row (S + 1) is never written by time-mix
    assert np.array_equal(gs[2], rs[2])
    assert np.array_equal(gs[:, S + 1], rs[:, S + 1])


@pytest.mark.parametrize("version", [5, 6])
def test_v56_decode_and_prefill(wrk, ctx, version):
    gx, gs, rx, rs = _v56_case(wrk, ctx, version, 32, [(0, 1)], 1, False, seed=10)
    assert_close(gx, rx, "decode x")
    assert_close(gs, rs, "decode state")
    gx, gs, rx, rs = _v56_case(wrk, ctx, version, 12, [(0, 96), (1, 32)], 2, True, seed=11)
    assert_close(gx, rx, "prefill x")
    assert_close(gs, rs, "prefill state")


def test_v6_fp16_io(wrk, ctx):
    gx, gs, rx, rs = _v56_case(wrk, ctx, 6, 4, [(0, 7), (1, 3)], 2, False, dtype=np.float16, seed=12)
    assert_close(gx, rx, "x f16")
    assert_close(gs, rs, "state")


def test_v6_packed_cursor_len_wraps_at_256(wrk, ctx):
    # 8-bit len: a 256-token run packs len = 0, so the token-shift carry is never written — the
    # packed form reproduces that, the wide form writes it (src/tensor/mod.rs:53-60)
    gx, gs, rx, rs = _v56_case(wrk, ctx, 6, 2, [(0, 256)], 1, False, seed=13)
    assert_close(gx, rx, "x")
    assert_close(gs, rs, "state")
    gxw, gsw, rxw, rsw = _v56_case(wrk, ctx, 6, 2, [(0, 256)], 1, True, seed=13)
    assert_close(gsw, rsw, "state wide")
    assert not np.array_equal(gs[0, 0], gsw[0, 0])  # carry row differs between the two forms


@pytest.mark.parametrize("head_size", [32, 128])
@pytest.mark.parametrize("version", [5, 6])
def test_v56_other_head_sizes(wrk, ctx, version, head_size):
    # runs that end inside, at the end of and past a staged chunk of tokens
    gx, gs, rx, rs = _v56_case(wrk, ctx, version, 3, [(0, 37), (1, 16), (2, 1)], 3, True, seed=40 + head_size, S=head_size)
    assert_close(gx, rx, "x")
    assert_close(gs, rs, "state")


@pytest.mark.parametrize("version", [5, 6])
@pytest.mark.parametrize("dtype", [np.float32, np.float16])
def test_v56_blocks_of_16_tokens(wrk, ctx, version, dtype):
    """The block form against the oracle's serial recurrence: runs shorter than, equal to and longer than a block, an idle
    slot, single tokens."""
    gx, gs, rx, rs = _v56_case(wrk, ctx, version, 5, [(1, 130), (0, 16), (3, 1), (4, 47)], 5, True, dtype=dtype, seed=60 + version,
                               blocks=True)
    assert_close(gx, rx, "x")
    assert_close(gs, rs, "state")
    assert np.array_equal(gs[2], rs[2])
    assert np.array_equal(gs[:, S + 1], rs[:, S + 1])


def test_v6_blocks_long_run_with_strong_decay(wrk, ctx):
    # 2048 tokens; decays down to exp(-e) per token, so that products over a block underflow towards zero
    gx, gs, rx, rs = _v56_case(wrk, ctx, 6, 2, [(0, 2048)], 1, True, seed=63, blocks=True)
    assert_close(gx, rx, "x")
    assert_close(gs, rs, "state")
    gx, gs, rx, rs = _v56_case(wrk, ctx, 6, 2, [(0, 256)], 1, False, seed=64, blocks=True)  # packed cursors: len wraps
    assert_close(gx, rx, "x packed")
    assert_close(gs, rs, "state packed")


def test_v6_long_runs_cross_chunks(wrk, ctx):
    gx, gs, rx, rs = _v56_case(wrk, ctx, 6, 5, [(1, 130), (0, 33), (2, 48)], 3, True, seed=44)
    assert_close(gx, rx, "x")
    assert_close(gs, rs, "state")


def _v7_case(wrk, ctx, H, seqs, B, wide, dtype=np.float16, seed=0, S=S):
    rng = np.random.default_rng(seed)
    C = S * H
    cursors, T = _cursors(seqs, wide)
    r = rng.standard_normal((T, H, S)).astype(dtype)
    w = rng.standard_normal((T, H, S)).astype(dtype)
    k = rng.standard_normal((T, H, S)).astype(np.float32)
    v = rng.standard_normal((T, H, S)).astype(np.float32)
    a = rng.uniform(0, 1, (T, H, S)).astype(np.float32)
    kk = rng.standard_normal((T, H, S)).astype(np.float32)
    kk /= np.linalg.norm(kk, axis=-1, keepdims=True)  # the model L2-normalises kk per head
    n = np.stack([k, v, a, kk]).astype(dtype)
    x = rng.standard_normal((T, H, S)).astype(dtype)
    state = (rng.standard_normal((B, S + 2, C)) * 0.1).astype(np.float32)

    t_state, t_x = ctx.from_numpy(state), ctx.from_numpy(x)
    op = wrk.time_mix_v7(ctx.from_numpy(cursors), t_state.view(y=(0, S + 1)), ctx.from_numpy(r), ctx.from_numpy(w),
                         ctx.from_numpy(n), t_x)
    ctx.run(op)
    got_x, got_state = t_x.numpy().reshape(T, H, S), t_state.numpy().reshape(B, S + 2, C)
    ref_x, ref_state = x.copy(), state.copy()
    oracle.time_mix_v7(cursors, oracle.View(ref_state, y=(0, S + 1)), r, w, n, ref_x, S, H)
    return got_x, got_state, ref_x, ref_state


@pytest.mark.parametrize("wide", [False, True])
@pytest.mark.parametrize("dtype", [np.float16, np.float32])
def test_v7_multi_sequence(wrk, ctx, wide, dtype):
    gx, gs, rx, rs = _v7_case(wrk, ctx, 4, [(1, 6), (2, 1), (3, 11)], 4, wide, dtype=dtype, seed=20)
    assert_close(gx, rx, "x")
    assert_close(gs, rs, "state")
    assert np.array_equal(gs[0], rs[0])


@pytest.mark.parametrize("head_size", [32, 128])
def test_v7_other_head_sizes(wrk, ctx, head_size):
    gx, gs, rx, rs = _v7_case(wrk, ctx, 3, [(0, 29), (1, 24), (2, 1)], 3, True, seed=50 + head_size, S=head_size)
    assert_close(gx, rx, "x")
    assert_close(gs, rs, "state")


@pytest.mark.parametrize("T", [1, 2, 64, 512])
def test_v7_sweep_64_heads(wrk, ctx, T):
    # the standalone sweep shape: 64 heads x 64x64 fp32 state, one sequence of T tokens
    gx, gs, rx, rs = _v7_case(wrk, ctx, 64, [(0, T)], 1, True, seed=T)
    assert_close(gx, rx, f"x T={T}")
    assert_close(gs, rs, f"state T={T}")


def test_v7_batched_decode(wrk, ctx):
    B = 64
    gx, gs, rx, rs = _v7_case(wrk, ctx, 8, [(b, 1) for b in range(B)], B, False, seed=30)
    assert_close(gx, rx, "x")
    assert_close(gs, rs, "state")


@pytest.mark.parametrize("dtype", [np.float16, np.float32])
def test_time_first_v7(wrk, ctx, dtype):
    rng = np.random.default_rng(40)
    H, T = 6, 5
    u = rng.uniform(0, 1, (H, S)).astype(np.float16)
    r = rng.standard_normal((T, H, S)).astype(dtype)
    n = rng.standard_normal((4, T, H, S)).astype(dtype)
    x = rng.standard_normal((T, H, S)).astype(dtype)
    t_x = ctx.from_numpy(x)
    ctx.run(wrk.time_first_v7(ctx.from_numpy(u), ctx.from_numpy(r), ctx.from_numpy(n), t_x))
    ref = x.copy()
    oracle.time_first_v7(u, r, n, ref, S, H)
    assert_close(t_x.numpy().reshape(T, H, S), ref, "time_first", max_abs=5e-2 if dtype == np.float16 else 2e-2)


def test_shape_errors(wrk, ctx):
    H, T = 2, 3
    f = lambda *s: ctx.tensor(wrk.F32, list(s))
    cursors = ctx.tensor(wrk.U32, [T])
    state = ctx.tensor(wrk.F32, [S * H, S + 2, 1])
    with pytest.raises(wrk.WrkError) as e:  # time_decay must be per token for v6
        wrk.time_mix_v6(cursors, f(S, H), f(S, H), state.view(y=(0, S + 1)), f(S, H, T), f(S, H, T), f(S, H, T),
                        f(S, H, T))
    assert e.value.status == -5
    with pytest.raises(wrk.WrkError) as e:  # state view must have S + 1 rows
        wrk.time_mix_v6(cursors, f(S, H, T), f(S, H), state, f(S, H, T), f(S, H, T), f(S, H, T), f(S, H, T))
    assert e.value.status == -5


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
def test_time_mix_v4(wrk, ctx, dtype):
    # TensorOp::time_mix_v4 (src/tensor/ops.rs:1464-1528): three sequences in three batch slots, one revisited slot
    rng = np.random.default_rng(44)
    C, B = 320, 3
    seqs = [(2, 0, 7), (0, 7, 1), (1, 8, 12)]
    T = 20
    k, v, r, x = (rng.standard_normal((T, C)).astype(dtype) for _ in range(4))
    w = (-np.exp(rng.uniform(-3, 0.5, C))).astype(np.float32)
    u = rng.uniform(-1, 1, C).astype(np.float32)
    state = rng.standard_normal((B, 4, C)).astype(np.float32)
    state[:, 2] = np.abs(state[:, 2]) + 0.5
    for wide in (True, False):
        cursors = oracle.pack_cursors(seqs, wide=wide)
        t_state, t_x = ctx.from_numpy(state), ctx.from_numpy(x)
        ctx.run(wrk.time_mix_v4(ctx.from_numpy(cursors), ctx.from_numpy(w), ctx.from_numpy(u), t_state,
                                ctx.from_numpy(k), ctx.from_numpy(v), ctx.from_numpy(r), t_x))
        x_ref, st_ref = x.copy(), state.copy()
        oracle.time_mix_v4(cursors, w, u, st_ref, k, v, r, x_ref)
        assert_close(t_x.numpy().reshape(T, C), x_ref, f"v4 x wide={wide}")
        assert_close(t_state.numpy().reshape(B, 4, C), st_ref, f"v4 state wide={wide}")
        assert np.array_equal(t_state.numpy().reshape(B, 4, C)[:, 0], st_ref[:, 0])  # the carry rows are copies
    with pytest.raises(wrk.WrkError) as e:
        wrk.time_mix_v4(ctx.from_numpy(cursors), ctx.from_numpy(w[:-4]), ctx.from_numpy(u), t_state, ctx.from_numpy(k),
                        ctx.from_numpy(v), ctx.from_numpy(r), t_x)
    assert e.value.status == -5
