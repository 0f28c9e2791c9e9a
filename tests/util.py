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
