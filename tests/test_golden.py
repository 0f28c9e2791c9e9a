"""Committed golden vectors (tests/golden/hotpath_small.npz, made by tests/golden/make_golden.py):
the CPU oracle must reproduce them here; on a GPU the CUDA kernels must match them too."""
import os

import numpy as np
import pytest

from oracle import oracle
from tests.util import assert_close

G = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "hotpath_small.npz"))
S, H = 64, 2


def test_oracle_reproduces_golden_quantizers():
    for src in ("w", "u"):
        q, mm = oracle.quantize_mat_int8(G[src])
        assert np.array_equal(q, G[f"{src}_int8"]) and np.array_equal(mm.view(np.uint16), G[f"{src}_minmax"].view(np.uint16))
        q, am = oracle.quantize_mat_nf4(G[src])
        assert np.array_equal(q, G[f"{src}_nf4"]) and np.array_equal(am.view(np.uint16), G[f"{src}_absmax"].view(np.uint16))


def test_oracle_reproduces_golden_matmul_and_wkv():
    for name, kind, q, s in (("int8", oracle.MAT_INT8, G["w_int8"], G["w_minmax"]),
                             ("nf4", oracle.MAT_NF4, G["w_nf4"], G["w_absmax"]), ("fp16", oracle.MAT_FP16, G["w"], None)):
        y = np.zeros((3, 48), dtype=np.float32)
        oracle.matmul(kind, q, s, G["x"], y)
        assert np.allclose(y, G[f"y_{name}"], rtol=0, atol=1e-6)
    x6, st6 = G["v6_x"].copy(), G["v6_state"].copy()
    oracle.time_mix_v56(True, G["cursors"], G["v6_w"], G["v6_u"], oracle.View(st6, y=(0, S + 1)), G["v6_k"], G["v6_v"],
                        G["v6_r"], x6, S, H)
    assert np.allclose(x6, G["v6_y"], atol=1e-6) and np.allclose(st6, G["v6_state_out"], atol=1e-6)
    y7, st7 = G["v7_x"].copy(), G["v6_state"].copy()
    oracle.time_mix_v7(G["cursors"], oracle.View(st7, y=(0, S + 1)), G["v7_r"], G["v7_w"], G["v7_n"], y7, S, H)
    assert np.array_equal(y7, G["v7_y"]) and np.allclose(st7, G["v7_state_out"], atol=1e-6)


@pytest.mark.gpu
def test_cuda_matches_golden(wrk, ctx):
    for src in ("w", "u"):
        t = ctx.from_numpy(G[src])
        _, w, m, _ = wrk.Matrix.quant_u8(t).parts()
        assert np.array_equal(w.numpy().reshape(G[f"{src}_int8"].shape), G[f"{src}_int8"])
        assert np.array_equal(m.numpy().reshape(-1).view(np.uint16), G[f"{src}_minmax"].view(np.uint16))
        _, w, m, _ = wrk.Matrix.quant_nf4(t).parts()
        assert np.array_equal(w.numpy().reshape(G[f"{src}_nf4"].shape), G[f"{src}_nf4"])
        assert np.array_equal(m.numpy().reshape(-1).view(np.uint16), G[f"{src}_absmax"].view(np.uint16))
    t_w, t_x = ctx.from_numpy(G["w"]), ctx.from_numpy(G["x"])
    for name, mat in (("int8", wrk.Matrix.quant_u8(t_w)), ("nf4", wrk.Matrix.quant_nf4(t_w)), ("fp16", wrk.Matrix.fp16(t_w))):
        t_y = ctx.tensor(wrk.F32, [48, 3])
        ctx.run(mat.matmul_op(t_x, t_y))
        assert_close(t_y.numpy().reshape(3, 48), G[f"y_{name}"], name)
    st = ctx.from_numpy(G["v6_state"])
    x6 = ctx.from_numpy(G["v6_x"])
    ctx.run(wrk.time_mix_v6(ctx.from_numpy(G["cursors"]), ctx.from_numpy(G["v6_w"]), ctx.from_numpy(G["v6_u"]),
                            st.view(y=(0, S + 1)), ctx.from_numpy(G["v6_k"]), ctx.from_numpy(G["v6_v"]),
                            ctx.from_numpy(G["v6_r"]), x6))
    assert_close(x6.numpy().reshape(G["v6_y"].shape), G["v6_y"], "v6 y")
    assert_close(st.numpy().reshape(G["v6_state_out"].shape), G["v6_state_out"], "v6 state")
    st = ctx.from_numpy(G["v6_state"])
    x7 = ctx.from_numpy(G["v7_x"])
    ctx.run(wrk.time_mix_v7(ctx.from_numpy(G["cursors"]), st.view(y=(0, S + 1)), ctx.from_numpy(G["v7_r"]),
                            ctx.from_numpy(G["v7_w"]), ctx.from_numpy(G["v7_n"]), x7))
    assert_close(x7.numpy().reshape(G["v7_y"].shape), G["v7_y"], "v7 y")
    assert_close(st.numpy().reshape(G["v7_state_out"].shape), G["v7_state_out"], "v7 state")
