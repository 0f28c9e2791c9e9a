"""Shared helpers of the parity tests."""
import numpy as np

# Tolerance of the floating-point part of the path: max-abs 2e-2 and cosine >= 0.9995 in fp16.
MAX_ABS = 2e-2
MIN_COS = 0.9995


def cosine(a, b):
    a = np.asarray(a, dtype=np.float64).ravel()
    b = np.asarray(b, dtype=np.float64).ravel()
    na, nb = np.linalg.norm(a), np.linalg.norm(b)
    if na == 0 and nb == 0:
        return 1.0
    return float(a @ b / (na * nb + 1e-300))


def assert_close(got, want, what="", max_abs=MAX_ABS, min_cos=MIN_COS):
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite values"
    # absolute for values up to 1, relative above (an fp16 result of magnitude 24 has an ulp of 0.016)
    err = float(np.max(np.abs(got - want) / np.maximum(1.0, np.abs(want)))) if got.size else 0.0
    cos = cosine(got, want)
    assert err <= max_abs, f"{what}: max-abs {err:.4g} > {max_abs}"
    assert cos >= min_cos, f"{what}: cosine {cos:.6f} < {min_cos}"


def assert_state_close(got, want, what=""):
    """Recurrent state (layers, S + 2, C) at real model widths.  A WKV matrix is a sum of k v products over all
    tokens seen: its entries span from near zero to ~100 at n_embd 4096, and an error that is small against the
    terms of the sum is not small against an entry that cancelled to 0.05.  An entry therefore passes within the
    path's tolerance (max-abs 2e-2, relative above 1) *or* within one fp16 spacing (2^-10) of the largest entry
    of the same layer's state; the cosine bar applies to the whole state as usual."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape and np.isfinite(got).all(), what
    for layer in range(want.shape[0]):
        err = np.abs(got[layer] - want[layer])
        bound = np.maximum(MAX_ABS * np.maximum(1.0, np.abs(want[layer])), 2.0 ** -10 * np.abs(want[layer]).max())
        worst = float((err / bound).max())
        assert worst <= 1.0, f"{what} layer {layer}: error {worst:.3g} x the bound (max |err| {err.max():.4g})"
    cos = cosine(got, want)
    assert cos >= MIN_COS, f"{what}: cosine {cos:.6f} < {MIN_COS}"


def is_approx_eps(a, b, eps):
    """The reference tests' comparison (src/tensor/ops.rs:2614-2618)."""
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return np.abs(a - b) <= np.maximum(eps, eps * np.maximum(np.abs(a), np.abs(b)))


def free_port():
    """A TCP port on the loopback interface that is free right now (for a torch.distributed rendezvous)."""
    import socket
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as sock:
        sock.bind(("127.0.0.1", 0))
        return sock.getsockname()[1]
