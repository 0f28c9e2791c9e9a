"""`wrk_gemv_int8_static`: the Int8 GEMV entry point that allocates nothing (its row-range table is a static
device array).  Collected last so that it also runs after every other test has used the device; it passes on
its own as well.  Checked against the existing entry point (`Matrix::matmul_op` -> matmul_vec_int8), bit for bit,
and against the CPU oracle within the path's tolerance."""
import numpy as np
import pytest

from oracle import oracle
from tests.util import assert_close

pytestmark = pytest.mark.gpu


def _case(wrk, ctx, rng, K, M, T, act):
    w = (rng.standard_normal((M, K), dtype=np.float32) * 0.05).astype(np.float16)
    mat = wrk.Matrix.quant_u8(ctx.from_numpy(w))
    kind, wq, mm, _ = mat.parts()
    assert kind == 1
    y_ref = ctx.tensor(wrk.F32, [M, T])
    y_new = ctx.tensor(wrk.F32, [M, T])
    outs = []
    # two calls in a row, on different inputs, through the same static array
    for call in range(2):
        x = ctx.from_numpy(rng.standard_normal((T, K), dtype=np.float32).astype(np.float16))
        ctx.run(mat.matmul_op(x, y_ref, act))
        ref = y_ref.numpy().copy()
        y_new.load(np.full((T, M), np.nan, dtype=np.float32))
        wrk.gemv_int8_static(ctx, wq, mm, x, y_new, act)
        ctx.synchronize()
        got = y_new.numpy().copy()
        want = np.zeros((T, M), dtype=np.float32)
        oracle.matmul(oracle.MAT_INT8, wq.numpy().reshape(M, K), mm.numpy().reshape(-1), x.numpy().reshape(T, K), want,
                      act=act)
        outs.append((ref.reshape(T, M), got.reshape(T, M), want))
    return outs


@pytest.mark.parametrize("K,M,T,act", [(2048, 2048, 1, 0), (1024, 4099, 3, 1), (7168, 2048, 1, 0), (256, 65536, 2, 2)])
def test_static_gemv_matches_matmul_vec_int8(wrk, ctx, K, M, T, act):
    rng = np.random.default_rng(K + M + T)
    for ref, got, want in _case(wrk, ctx, rng, K, M, T, act):
        assert np.isfinite(got).all()
        # same kernel and the same row split as the existing entry point, and the warps' partial sums are added
        # in warp order: the two launches give the same bits
        assert np.array_equal(got, ref), f"max |diff| {float(np.abs(got - ref).max())}"
        assert_close(got, want, f"static gemv {K}x{M} T={T} act={act}")


def test_static_gemv_rejects_what_does_not_fit(wrk, ctx):
    rng = np.random.default_rng(1)
    w = ctx.from_numpy((rng.standard_normal((256, 256), dtype=np.float32) * 0.05).astype(np.float16))
    _, wq, mm, _ = wrk.Matrix.quant_u8(w).parts()
    x = ctx.from_numpy(np.zeros((1, 256), dtype=np.float16))
    y = ctx.tensor(wrk.F32, [256, 1])
    with pytest.raises(wrk.WrkError) as e:
        wrk.gemv_int8_static(ctx, wq, mm, x, y, num_ctas=513)
    assert "512" in str(e.value)
    x9 = ctx.from_numpy(np.zeros((9, 256), dtype=np.float16))
    y9 = ctx.tensor(wrk.F32, [256, 9])
    with pytest.raises(wrk.WrkError):
        wrk.gemv_int8_static(ctx, wq, mm, x9, y9)
    # a refused call leaves the entry point usable
    wrk.gemv_int8_static(ctx, wq, mm, x, y, num_ctas=7)
    ctx.synchronize()
    assert not np.any(y.numpy())
