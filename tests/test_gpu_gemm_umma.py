"""Tensor-memory GEMM (matmul_mat_* with 16 or more tokens) against the CPU oracle: token counts around the
tile sizes, ragged row counts, split-K shapes (clusters of 4, 7 and 8 CTAs that add their partial tiles through
distributed shared memory), output types, activations, views, and repeated launches.  Tolerance: tests/util.py."""
import numpy as np
import pytest

from oracle import oracle
from tests.test_gpu_matmul import KINDS, _make_matrix, _run
from tests.util import assert_close

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kind", KINDS)
@pytest.mark.parametrize("n", [16, 31, 100, 256, 257, 600])
def test_token_counts_around_the_tiles(wrk, ctx, kind, n):
    got, want = _run(wrk, ctx, kind, 1024, 384, n, turbo=(n % 32 == 0), seed=n)
    assert_close(got, want, f"{kind} n={n}")


@pytest.mark.parametrize("kind", KINDS)
@pytest.mark.parametrize("k,m,n", [(2048, 256, 64), (4096, 128, 32), (2048, 2048, 256), (512, 4099, 48), (7168, 300, 128)])
def test_split_k_and_ragged_rows(wrk, ctx, kind, k, m, n):
    # few output tiles and a long K: K is split over a cluster (4, 8, 4 with 128-token tiles, none, 7 CTAs);
    # 4099 / 300 rows: last tile ragged
    got, want = _run(wrk, ctx, kind, k, m, n, turbo=True, seed=k + m + n)
    assert_close(got, want, f"{kind} {k}x{m} n={n}")


@pytest.mark.parametrize("kind", KINDS)
def test_fp16_output_and_activation(wrk, ctx, kind):
    got, want = _run(wrk, ctx, kind, 1024, 512, 64, turbo=True, out_dt=np.float16, act=1, seed=3)  # squared relu
    assert_close(got, want, f"{kind} f16 out, squared relu")
    got, want = _run(wrk, ctx, kind, 1024, 512, 64, turbo=True, act=2, seed=4)  # tanh
    assert_close(got, want, f"{kind} tanh")


def test_repeated_split_k_launches(wrk, ctx):
    rng = np.random.default_rng(11)
    w = (rng.standard_normal((256, 2048), dtype=np.float32) * 0.02).astype(np.float16)
    mat, (okind, om, oscale) = _make_matrix(wrk, ctx, "int8", w)
    y = ctx.tensor(wrk.F32, [256, 64])
    for rep in range(3):
        x = rng.standard_normal((64, 2048), dtype=np.float32).astype(np.float16)
        ctx.run(mat.matmul_op(ctx.from_numpy(x), y, turbo=True))
        want = np.zeros((64, 256), dtype=np.float32)
        oracle.matmul(okind, om, oscale, x, want, mode=1)
        assert_close(y.numpy().reshape(64, 256), want, f"launch {rep}")
    assert ctx.device_status() == 0


def test_activation_view_with_row_stride(wrk, ctx):
    # activations taken as a z-slice of a [K, N, 3] tensor (as the v6 layer does with its five shifted inputs)
    rng = np.random.default_rng(12)
    K, M, N = 1024, 256, 64
    w = (rng.standard_normal((M, K), dtype=np.float32) * 0.02).astype(np.float16)
    mat, (okind, om, oscale) = _make_matrix(wrk, ctx, "nf4", w)
    x3 = rng.standard_normal((3, N, K), dtype=np.float32).astype(np.float16)
    t_x = ctx.from_numpy(x3)
    y = ctx.tensor(wrk.F32, [M, N])
    ctx.run(mat.matmul_op(t_x.view(z=2), y, turbo=True))
    want = np.zeros((N, M), dtype=np.float32)
    oracle.matmul(okind, om, oscale, np.ascontiguousarray(x3[2]), want, mode=1)
    assert_close(y.numpy().reshape(N, M), want, "z-slice input")
