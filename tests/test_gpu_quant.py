"""Int8 / NF4 packing: CUDA kernels against the CPU oracle, bit for bit, through the C ABI.

Shapes follow the reference's own tests (src/tensor/ops.rs:3058-3059, 3253-3254) plus ragged,
degenerate and full-size cases.
"""
import numpy as np
import pytest

from oracle import oracle

pytestmark = pytest.mark.gpu


def _int8_roundtrip(wrk, ctx, m):
    K = m.shape[-1]
    t_in = ctx.from_numpy(m)
    t_out = ctx.tensor(wrk.U8, wrk.np_to_shape(m))
    t_mm = ctx.tensor(wrk.F16, [2 * ((m.size + 127) // 128)])
    ctx.run(wrk.quantize_mat_int8(t_in, t_mm, t_out))
    return t_out.numpy().reshape(m.shape), t_mm.numpy().reshape(-1)


def _nf4_roundtrip(wrk, ctx, m, table=None):
    table = oracle.NF4_TABLE if table is None else table
    t_in = ctx.from_numpy(m)
    shape = wrk.np_to_shape(m)
    shape[0] //= 2
    t_out = ctx.tensor(wrk.U8, shape)
    t_am = ctx.tensor(wrk.F16, [(m.size + 63) // 64])
    t_q = ctx.from_numpy(np.asarray(table, dtype=np.float32))
    ctx.run(wrk.quantize_mat_nf4(t_in, t_q, t_am, t_out))
    return t_out.numpy().reshape(m.shape[:-1] + (m.shape[-1] // 2,)), t_am.numpy().reshape(-1)


@pytest.mark.parametrize("c,r", [(2560, 2048), (320, 64), (128, 4), (2048, 7168)])
def test_int8_bit_exact(wrk, ctx, c, r):
    rng = np.random.default_rng(42 + c + r)
    m = (10.0 * (rng.random((r, c), dtype=np.float32) - 0.5)).astype(np.float16)
    q, mm = _int8_roundtrip(wrk, ctx, m)
    q_ref, mm_ref = oracle.quantize_mat_int8(m)
    assert np.array_equal(mm.view(np.uint16), mm_ref.view(np.uint16))
    assert np.array_equal(q, q_ref)


def test_int8_weights_distribution_and_edges(wrk, ctx):
    rng = np.random.default_rng(7)
    m = (rng.standard_normal((64, 512)) * 0.02).astype(np.float16)
    m[0, :128] = 0.25          # degenerate block: max == min
    m[1, :128] = 0.0           # all-zero block
    m[2, 0] = 65504.0          # f16 max
    m[2, 1] = -65504.0
    m[3, :4] = [1e-7, -1e-7, 6e-8, 0.0]  # subnormals
    q, mm = _int8_roundtrip(wrk, ctx, m)
    q_ref, mm_ref = oracle.quantize_mat_int8(m)
    assert np.array_equal(mm.view(np.uint16), mm_ref.view(np.uint16))
    assert np.array_equal(q, q_ref)
    assert (q[0, :128] == 0).all() and (q[1, :128] == 0).all()


def test_int8_ragged_length(wrk, ctx):
    # total length not a multiple of 128 nor of 8: the last block is short
    rng = np.random.default_rng(3)
    m = rng.standard_normal((3, 100)).astype(np.float16)
    q, mm = _int8_roundtrip(wrk, ctx, m)
    q_ref, mm_ref = oracle.quantize_mat_int8(m)
    assert np.array_equal(mm.view(np.uint16), mm_ref.view(np.uint16))
    assert np.array_equal(q, q_ref)


@pytest.mark.parametrize("c,r", [(2560, 2048), (320, 64), (64, 8), (2560, 8960)])
def test_nf4_bit_exact(wrk, ctx, c, r):
    rng = np.random.default_rng(4242 + c + r)
    m = rng.standard_normal((r, c)).astype(np.float16)
    q, am = _nf4_roundtrip(wrk, ctx, m)
    q_ref, am_ref = oracle.quantize_mat_nf4(m)
    assert np.array_equal(am.view(np.uint16), am_ref.view(np.uint16))
    assert np.array_equal(q, q_ref)


def test_nf4_ties_and_edges(wrk, ctx):
    table = oracle.NF4_TABLE
    m = np.zeros((8, 64), dtype=np.float16)
    m[0, :] = 0.0                      # all-zero block: 1/0 = inf, 0 * inf = NaN → index 0
    m[1, 0] = 1.0                      # absmax 1: exact table values and midpoints
    m[1, 1:17] = table.astype(np.float16)[:16]
    mids = ((table[:-1] + table[1:]) / 2).astype(np.float16)
    m[1, 17:32] = mids
    m[2, 0] = 3.0
    m[2, 1:16] = (3.0 * mids.astype(np.float32)).astype(np.float16)
    m[3, :] = np.linspace(-2, 2, 64).astype(np.float16)
    m[4, :] = 65504.0
    m[5, :] = -6e-8
    rng = np.random.default_rng(9)
    m[6:, :] = (rng.standard_normal((2, 64)) * 0.02).astype(np.float16)
    q, am = _nf4_roundtrip(wrk, ctx, m)
    q_ref, am_ref = oracle.quantize_mat_nf4(m)
    assert np.array_equal(am.view(np.uint16), am_ref.view(np.uint16))
    assert np.array_equal(q, q_ref)


def test_nf4_unsorted_table_uses_literal_scan(wrk, ctx):
    rng = np.random.default_rng(11)
    table = oracle.NF4_TABLE.copy()
    rng.shuffle(table)
    m = rng.standard_normal((32, 128)).astype(np.float16)
    q, am = _nf4_roundtrip(wrk, ctx, m, table)
    q_ref, am_ref = oracle.quantize_mat_nf4(m, table)
    assert np.array_equal(q, q_ref)
    assert np.array_equal(am.view(np.uint16), am_ref.view(np.uint16))


@pytest.mark.parametrize("nu", [5.0, 2.0])
def test_sf4_matrix_bit_exact(wrk, ctx, nu):
    # Matrix::quant_sf4 (src/tensor/matrix.rs:202-222): the Fp4 packing with the Student-t code book
    rng = np.random.default_rng(int(nu * 10))
    m = (rng.standard_t(5.0, size=(64, 512)) * 0.02).astype(np.float16)
    table = wrk.sf4_table(nu)
    assert np.array_equal(table, oracle.sf4_table(nu))
    kind, w, am, q = wrk.Matrix.quant_sf4(ctx.from_numpy(m), nu).parts()
    q_ref, am_ref = oracle.quantize_mat_nf4(m, table)
    assert np.array_equal(q.numpy().reshape(-1), table)
    assert np.array_equal(w.numpy().reshape(q_ref.shape), q_ref)
    assert np.array_equal(am.numpy().reshape(-1).view(np.uint16), am_ref.view(np.uint16))


def test_full_size_checksum(wrk, ctx):
    # 7B-shaped FFN matrix (4096 x 14336): compare every byte with the oracle
    rng = np.random.default_rng(2024)
    m = (rng.standard_normal((4096, 14336), dtype=np.float32) * 0.02).astype(np.float16)
    q, mm = _int8_roundtrip(wrk, ctx, m)
    q_ref, mm_ref = oracle.quantize_mat_int8(m)
    assert np.array_equal(q, q_ref) and np.array_equal(mm.view(np.uint16), mm_ref.view(np.uint16))
    q4, am = _nf4_roundtrip(wrk, ctx, m)
    q4_ref, am_ref = oracle.quantize_mat_nf4(m)
    assert np.array_equal(q4, q4_ref) and np.array_equal(am.view(np.uint16), am_ref.view(np.uint16))


def test_shape_errors(wrk, ctx):
    t_in = ctx.tensor(wrk.F16, [256, 4])
    t_out = ctx.tensor(wrk.U8, [256, 4])
    bad = ctx.tensor(wrk.F16, [7])
    with pytest.raises(wrk.WrkError) as e:
        wrk.quantize_mat_int8(t_in, bad, t_out)
    assert e.value.status == -5  # TensorErrorKind::Shape
    with pytest.raises(wrk.WrkError) as e:
        wrk.quantize_mat_int8(t_out, bad, t_out)
    assert e.value.status == -2  # TensorErrorKind::Type
