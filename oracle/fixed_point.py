"""TEST INFRASTRUCTURE (never on a product path): a numpy restatement of the fixed-point activation rows that the
int8 tensor-core GEMV builds in shared memory (ingot_b200/csrc/pack.cuh: fx_store), and of a projection computed
from them.  The reference has no such rows — its kernels multiply float activations (kernels/generic.metal:182-313,
kernels/iq3_mix.metal:85-128) — so what this file pins is that the only approximation the rows introduce, one
rounding of every activation to 16 or 32 bits of fixed point under a power-of-two scale per 32 columns, keeps a
projection inside the reference's bound (tests/projections.rs:42-46).  The integer sums of the kernel are exact, so
a projection here is the float64 dot of the dequantised weights with the rounded activations."""
import numpy as np


def quantise_rows(x: np.ndarray, digits: int):
    """x [cols] float32 -> (xq int64 [cols], inv float32 [cols / 32]): per 32 columns the scale S = 2^k that puts the
    largest magnitude into [2^(LB-1), 2^LB) (LB = 15 for two digits, 30 for four; one step less when the two-digit
    rounding would leave the int8 range of the high digit), xq = rint(x * S) evaluated in float32, inv = 1 / S.
    A sub-block whose largest magnitude has a biased exponent below 32 keeps S = 1; non-finite values poison inv."""
    assert digits in (2, 4) and x.size % 32 == 0
    lb = 15 if digits == 2 else 30
    x = np.ascontiguousarray(x, np.float32).reshape(-1, 32)
    m = np.abs(x).max(axis=1)
    e = (m.view(np.uint32) >> 23).astype(np.int64)
    s = np.ones(len(m), np.float32)
    inv = np.ones(len(m), np.float32)
    ok = (e >= 32) & (e < 255)
    se = 253 + lb - e
    if digits == 2:
        with np.errstate(over="ignore", invalid="ignore"):
            trial = m * (np.where(ok, se, 127).astype(np.uint32) << 23).view(np.float32)
        se = np.where(ok & (trial > np.float32(32512.0)), se - 1, se)
    s[ok] = (se[ok].astype(np.uint32) << 23).view(np.float32)
    inv[ok] = ((254 - se[ok]).astype(np.uint32) << 23).view(np.float32)
    inv[e == 255] = m[e == 255]
    inv[np.isnan(x).any(axis=1)] = np.float32(np.nan)
    with np.errstate(over="ignore", invalid="ignore"):
        xq = np.rint(x * s[:, None])
    return xq.reshape(-1), inv


def digits_of(xq: np.ndarray, digits: int) -> np.ndarray:
    """The signed base-256 digits the kernel stores, most significant first: value = sum d_k 256^(digits-1-k), every
    digit in [-128, 127] (a digit above 127 carries into the next one)."""
    r = np.asarray(xq, np.int64).copy()
    out = np.zeros((digits, r.size), np.int64)
    for d in range(digits - 1, -1, -1):
        low = ((r + 128) & 0xFF) - 128
        out[d] = low
        r = (r - low) >> 8
    assert (r == 0).all(), "value does not fit the digits"
    return out


def project(weights: np.ndarray, x: np.ndarray, digits: int) -> np.ndarray:
    """weights [rows][cols] (dequantised, float64), x [cols] float32: the projection from fixed-point rows, with exact
    sums per 32 columns and the sub-block's 1/S applied to each."""
    xq, inv = quantise_rows(x, digits)
    rows, cols = weights.shape
    part = (weights.reshape(rows, cols // 32, 32) * xq.reshape(1, cols // 32, 32)).sum(axis=2)
    return (part * inv.astype(np.float64)[None, :]).sum(axis=1)
