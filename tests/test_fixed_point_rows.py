"""The fixed-point activation rows of the int8 GEMV, restated in numpy (oracle/fixed_point.py), on the CPU: the
rounding they introduce keeps a projection inside the reference's bound for every format, bfloat16-rounded inputs
are carried exactly by two digits, and the digit split the kernel stores reassembles the value."""
import numpy as np
import pytest

from ingot_b200 import Q4_0, Q4_K, Q6_K, Q8_0, synth
from oracle import fixed_point as FX
from oracle import oracle as O


def tol_ref_scaled(e):
    rms = float(np.sqrt(np.mean(np.square(e)))) if e.size else 0.0
    return 1e-4 * max(1.0, rms) + 5e-5 * np.abs(e)


@pytest.mark.parametrize("kind,cols,rows", [(Q4_K, 4096, 64), (Q6_K, 12288, 24), (Q4_0, 2560, 40), (Q8_0, 1024, 33)])
@pytest.mark.parametrize("digits,bf16", [(2, True), (4, False)])
def test_projection_from_fixed_point_rows_meets_the_reference_bound(kind, cols, rows, digits, bf16):
    raw = synth.random_matrix(kind, cols, rows, seed=cols + rows)
    w = O.dequant(raw, cols, rows, kind).reshape(rows, cols).astype(np.float64)

    def worst(x):
        if bf16:
            x = synth.from_bf16_bits(synth.to_bf16_bits(x))
        got = FX.project(w, x, digits)
        want = O.matvec_f64(raw, cols, rows, kind, x.reshape(1, cols))[0]
        return float((np.abs(got - want) / tol_ref_scaled(want)).max())

    x = synth.activations(1, cols, seed=digits)[0]
    x[64:96] = 0.0                                    # an all-zero sub-block keeps S = 1
    x[130] = np.float32(1e-30)                        # far below its sub-block's largest value: rounds to zero
    # well-scaled activations: the rounding to 15 (30) bits under the sub-block's scale is a small part of the bound
    assert worst(x.copy()) <= (0.25 if digits == 2 else 0.01)
    # an outlier coarsens its own 32 columns only.  30 times its neighbours: still inside the bound.  300 times: with
    # two digits the neighbours keep about 7 bits (bfloat16 carries 8) and a projection can leave the reference's
    # bound by a factor below two (measured here: 0.6 to 1.7 over the four formats); four digits (float32 rows) are
    # not affected.  The design document states this limit of the two-digit rows.
    y = x.copy()
    y[7] *= 30.0
    assert worst(y) <= (0.6 if digits == 2 else 0.01)
    x[7] *= 300.0
    assert worst(x) <= (2.0 if digits == 2 else 0.01)


def test_bfloat16_values_near_the_sub_block_maximum_are_exact_in_two_digits():
    rng = np.random.default_rng(3)
    x = synth.from_bf16_bits(synth.to_bf16_bits(rng.uniform(0.5, 1.0, 64).astype(np.float32) * np.float32(3.0)))
    xq, inv = FX.quantise_rows(x, 2)
    assert np.array_equal((xq * np.repeat(inv, 32)).astype(np.float32), x)      # 8 significant bits inside 15
    assert (np.abs(xq) < 32768).all() and (np.abs(xq).reshape(-1, 32).max(axis=1) >= 8192).all()


@pytest.mark.parametrize("digits", [2, 4])
def test_digits_reassemble_and_stay_in_int8(digits):
    rng = np.random.default_rng(digits)
    x = rng.normal(0, 1, 4096).astype(np.float32) * np.float32(17.0)
    x[:32] = np.float32(-1.0)                         # -2^14 / -2^29 exactly: the most negative values of a sub-block
    xq, _ = FX.quantise_rows(x, digits)
    d = FX.digits_of(xq, digits)
    assert d.min() >= -128 and d.max() <= 127
    assert np.array_equal(sum(d[k] * 256 ** (digits - 1 - k) for k in range(digits)), xq.astype(np.int64))


def test_non_finite_activations_poison_their_sub_block_only():
    x = np.ones(96, np.float32)
    x[40] = np.inf
    x[70] = np.nan
    _, inv = FX.quantise_rows(x, 2)
    assert np.isfinite(inv[0]) and np.isinf(inv[1]) and np.isnan(inv[2])
