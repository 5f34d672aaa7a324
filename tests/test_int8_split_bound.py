"""The two-term int8 form of the activations that the Q4_0 gate/up product uses at decode
(x ~ sx * (q0 + q1 / 254) per 32-input block, sx = amax / 127; built on the device by
dcommon::build_xq_block): a numpy restatement and its error bound, amax / (127 * 508)."""
import numpy as np


def split_two_terms(x):
    x = x.reshape(-1, 32).astype(np.float32)
    amax = np.abs(x).max(axis=1, keepdims=True)
    inv = (np.float32(127.0) / np.where(amax > 0, amax, np.float32(1.0))).astype(np.float32) * (amax > 0)
    sx = (amax * np.float32(1.0 / 127.0)).astype(np.float32)
    r = (x * inv).astype(np.float32)
    q0 = np.rint(r)
    q1 = np.rint(((r - q0) * np.float32(254.0)).astype(np.float32))
    return sx.astype(np.float64), q0.astype(np.float64), q1.astype(np.float64), amax.astype(np.float64)


def test_terms_fit_int8_and_error_bound():
    rng = np.random.default_rng(0)
    for scale in (1e-6, 1.0, 300.0):
        x = (rng.standard_normal(32 * 4096) * scale).astype(np.float32)
        x[:32] = 0.0                      # an all-zero block
        x[32:64] = scale                  # a constant block (every value at amax)
        sx, q0, q1, amax = split_two_terms(x)
        assert np.abs(q0).max() <= 127 and np.abs(q1).max() <= 127
        rec = sx * (q0 + q1 / 254.0)
        err = np.abs(rec - x.reshape(-1, 32).astype(np.float64))
        bound = amax / (127.0 * 508.0)
        # 1 % of slack for the f32 roundings of 127 / amax and x * (127 / amax) on the device
        assert np.all(err <= bound * 1.01 + 1e-30)
        assert np.all(rec[0] == 0.0)


def test_offset_term_removes_the_unsigned_nibble_bias():
    # sum_k (n_k - 8) * x_k == sum_k n_k * x_k - 8 * sum_k x_k: with x replaced by its two-term form the
    # second sum is the per-block value {8 * sx * sum(q0 + q1 / 254)} that rides with the scale
    rng = np.random.default_rng(1)
    x = rng.standard_normal(32).astype(np.float32)
    n = rng.integers(0, 16, 32)
    sx, q0, q1, _ = split_two_terms(x)
    xq = sx[0, 0] * (q0[0] + q1[0] / 254.0)
    lhs = np.sum((n - 8) * xq)
    raw = sx[0, 0] * (np.sum(n * q0[0]) + np.sum(n * q1[0]) / 254.0)
    off = 8.0 * sx[0, 0] * np.sum(q0[0] + q1[0] / 254.0)
    assert abs(lhs - (raw - off)) < 1e-9
