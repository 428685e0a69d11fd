"""Shared helpers of the test-suite: seeded inputs and error metrics."""
import numpy as np


def seeded_values(seed: int, length: int) -> np.ndarray:
    """The xorshift generator of the reference's tests/cpu_reference_oracle.rs:18-36."""
    mask = (1 << 64) - 1
    state = seed
    out = np.empty(length, dtype=np.float32)
    for i in range(length):
        state ^= (state << 13) & mask
        state ^= state >> 7
        state ^= (state << 17) & mask
        hi = (state >> 32) & 0xFFFFFFFF
        as_i32 = hi - (1 << 32) if hi >= (1 << 31) else hi
        rem = abs(as_i32) % 2049
        rem = -rem if as_i32 < 0 else rem  # Rust `%` keeps the dividend's sign
        centered = np.float32(rem - 1024) / np.float32(256.0)
        bias = (-0.75, -0.25, 0.0, 0.25, 0.75)[i % 5]
        out[i] = np.float32(centered) + np.float32(bias)
    return out


def normal(seed, shape, sigma):
    rng = np.random.Generator(np.random.Philox(seed))
    return (rng.standard_normal(shape, dtype=np.float32) * np.float32(sigma)).astype(np.float32)


def max_err_vs_rms(got: np.ndarray, want: np.ndarray) -> float:
    """max |got - want| divided by the RMS of `want` (the output's L2 norm per element)."""
    want = want.astype(np.float64)
    rms = np.sqrt(np.mean(want ** 2))
    return float(np.max(np.abs(got.astype(np.float64) - want)) / max(rms, 1e-30))


def assert_close(label, actual, expected, abs_tol, rel_tol):
    """tests/cpu_reference_oracle.rs:81-91."""
    actual, expected = np.asarray(actual).ravel(), np.asarray(expected).ravel()
    assert actual.shape == expected.shape, f"{label}: length mismatch"
    allowed = np.maximum(abs_tol, np.abs(expected) * rel_tol)
    err = np.abs(actual - expected)
    bad = np.nonzero(err > allowed)[0]
    assert bad.size == 0, (f"{label}[{bad[0]}] mismatch: got {actual[bad[0]]}, "
                           f"expected {expected[bad[0]]}")
