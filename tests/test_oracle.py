"""The oracle against its pins: the golden vectors produced by the reference's own
decoders, the reference's closed-form test fixtures, and (where the reference tree
is mounted) the reference decoders themselves."""
import glob
import os

import numpy as np
import pytest

from conftest import Lcg, lcg_q4k_fixture, q4_0_hand_expected, q4_0_hand_fixture, standard_x, tol_ref
from ingot_b200 import synth
from oracle import oracle as O

GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "decode_kind*.npz")))


def test_golden_files_present():
    assert len(GOLDEN) == 7


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p) for p in GOLDEN])
def test_oracle_matches_reference_golden_bits(path):
    g = np.load(path)
    got = O.dequant(g["raw"], int(g["cols"]), int(g["rows"]), int(g["kind"]))
    assert np.array_equal(got.view(np.uint32), g["expected_bits"])
    assert int(g["gguf_equal"]) in (-1, 1)      # gguf-py agreed when the fixture was made


@pytest.mark.skipif(not O.ref_available(), reason="reference tree not mounted; oracle/_ref not built")
@pytest.mark.parametrize("kind", [0, 1, 2, 8, 12, 14, 30])
def test_oracle_matches_reference_decoder_live(kind):
    raw = synth.random_matrix(kind, 1024, 9, seed=77 + kind)
    a = O.dequant(raw, 1024, 9, kind)
    r = O.ref_dequant(raw, 1024, 9, kind)
    assert np.array_equal(a.view(np.uint32), r.view(np.uint32))


def test_geometry_table():
    # src/gguf.rs:470-491
    assert [O.geometry(k) for k in (0, 1, 30, 2, 8, 12, 14)] == [(1, 4), (1, 2), (1, 2), (32, 18), (32, 34),
                                                                (256, 144), (256, 210)]
    with pytest.raises(ValueError):
        O.geometry(13)
    assert O.stride_of(12, 4096) == 2304 and O.stride_of(14, 12288) == 10080 and O.stride_of(2, 2560) == 1440


def test_invalid_layouts_rejected():
    with pytest.raises(ValueError):
        O.dequant(np.zeros(143, np.uint8), 256, 1, 12)
    with pytest.raises(ValueError):
        O.stride_of(12, 255)


def test_f32_matmul_tails_and_expert_offset_closed_form():
    # src/metal/tests.rs:14-34: value i/32+1, expert 1, expectation (rows + r + 1)*32*(t+1)
    for rows in (1, 3, 4, 5, 7, 33):
        raw = np.array([i // 32 + 1 for i in range(2 * rows * 32)], dtype=np.float32).view(np.uint8)
        for count in (1, 2, 4, 5, 8):
            x = np.array([i // 32 + 1 for i in range(32 * count)], dtype=np.float32)
            y = O.matvec_f64(raw, 32, rows, 0, x, expert=1)
            exp = np.array([[(rows + r + 1) * 32 * (t + 1) for r in range(rows)] for t in range(count)], float)
            assert np.abs(y - exp).max() < 2e-5


def test_q4_0_hand_fixture_closed_form():
    # src/metal/tests.rs:36-93
    rows, cols, experts, top = 7, 64, 5, 3
    data = q4_0_hand_fixture(rows, cols, experts)
    assert data.size == rows * experts * 36
    for tokens in (1, 2, 3, 5, 8):
        pairs = tokens * top
        ids = [(i * 7 + 1) % experts for i in range(pairs)]
        for per in (False, True):
            n_in = cols * (pairs if per else tokens)
            inputs = np.array([(i % 19) * 0.125 - 1.0 for i in range(n_in)], dtype=np.float32)
            exp = q4_0_hand_expected(ids, rows, cols, top, per, inputs)
            for pair in range(pairs):
                inp = pair if per else pair // top
                y = O.matvec_f64(data, cols, rows, 2, inputs[inp * cols:(inp + 1) * cols], expert=ids[pair])
                assert np.abs(y[0] - exp[pair]).max() < 2e-5


def test_route_known_answers():
    # src/main.rs:341-349
    ids, w = O.route([1000.0, -1000.0, 1000.0, 999.0], 3)
    assert ids.tolist() == [0, 2, 3]
    assert abs(float(w.sum()) - 1.0) < 1e-6
    assert abs(float(w[0] / w[2]) - np.e) < 1e-5
    for bad in (([1.0, float("nan")], 1), ([1.0, 2.0], 0), ([1.0, 2.0], 3), ([float("inf"), 0.0], 1)):
        with pytest.raises(ValueError):
            O.route(*bad)


@pytest.mark.parametrize("count", [1, 31, 33, 288, 512])
@pytest.mark.parametrize("ties", [False, True])
def test_route_matches_stable_sort(count, ties):
    # src/metal/tests.rs:95-137: the CPU rule is a stable descending sort (src/lib.rs:47-50)
    logits = np.array([1000.0 if ties else float((i * 17) % 23) - 11.0 for i in range(count)], np.float32)
    top = min(count, 10)
    ids, w = O.route(logits, top)
    order = sorted(range(count), key=lambda i: -logits[i])[:top]       # Python's sort is stable
    assert ids.tolist() == order
    ref = np.exp(logits[order] - logits[order[0]]).astype(np.float32)
    assert np.abs(w - ref / ref.sum()).max() < 2e-6


def test_lcg_q4k_fixture_properties():
    # src/expert_bench.rs:652-688: f16 scales forced into [0x1c00, 0x1c00+2560)
    g = Lcg(23)
    first = g.next()
    assert 0.0 <= first < 1.0
    data = lcg_q4k_fixture(cols=512, rows=3, experts=1)
    bits = data.reshape(-1, 144)[:, :4].copy().view(np.uint16)
    assert bits.min() >= 0x1C00 and bits.max() < 0x1C00 + 2560
    w = O.dequant(data, 512, 3, 12)
    assert np.isfinite(w).all()
    x = standard_x(512)
    assert np.abs(O.matvec_f32(data, 512, 3, 12, x) - O.matvec_f64(data, 512, 3, 12, x)).max() < tol_ref(
        O.matvec_f64(data, 512, 3, 12, x)).min() * 10


def test_f16_roundtrip_and_gemm_rounding():
    vals = np.array([0.0, 1.0, -2.5, 65504.0, 1e-8, 6.1e-5, 3.14159, 70000.0, -1e-10], np.float32)
    ours = np.array([O.lib().oracle_half_to_float(O.lib().oracle_float_to_half(float(v))) for v in vals], np.float32)
    with np.errstate(over="ignore"):
        theirs = vals.astype(np.float16).astype(np.float32)
    assert np.array_equal(ours.view(np.uint32), theirs.view(np.uint32))
    raw = synth.random_matrix(12, 512, 4, seed=3)
    x = standard_x(512 * 2).reshape(2, 512)
    exact, rounded = O.matvec_f64(raw, 512, 4, 12, x), O.gemm_f16_f64(raw, 512, 4, 12, x)
    assert np.abs(exact - rounded).max() > 0 and np.abs(exact - rounded).max() < 2e-3 * np.abs(exact).max()


def test_glu_and_moe_glue():
    g, u = np.array([0.5, -1.25, 3.0], np.float32), np.array([2.0, 0.5, -1.0], np.float32)
    assert np.allclose(O.glu(g, u), g / (1 + np.exp(-g)) * u, rtol=1e-6)
    t = np.tanh(0.7978845608 * g * (1 + 0.044715 * g * g))
    assert np.allclose(O.glu(g, u, gelu=True), 0.5 * g * (1 + t) * u, rtol=1e-6)
    routed = np.arange(2 * 3 * 4, dtype=np.float32).reshape(6, 4)
    w = np.array([0.5, 0.25, 0.25, 0.1, 0.2, 0.7], np.float32)
    y = O.moe_sum(routed, w, 4, 3)
    assert np.allclose(y[1], (routed[3:6] * w[3:6, None]).sum(0))
    out = O.combine(routed[:3], np.ones(4, np.float32), w[:3], 0.0, 4)
    assert np.allclose(out, (routed[:3] * w[:3, None]).sum(0) + 0.5)


def test_expert_layout_is_stable_and_tiled():
    # kernels/prefill.metal:7-35: experts ascending, pairs ascending inside, 32-pair tiles
    rng = np.random.default_rng(5)
    ids = rng.integers(0, 6, 100).astype(np.uint32)
    ids[:40] = 2
    layout, tiles, pairs, inverse, n = O.expert_layout(ids, 6, 16)
    assert layout[:, 0].sum() == 100
    at = 0
    for e in range(6):
        idx = np.nonzero(ids == e)[0]
        assert layout[e].tolist() == [len(idx), at]
        assert pairs[at:at + len(idx)].tolist() == idx.tolist()
        at += len(idx)
    assert np.array_equal(pairs[inverse], np.arange(100))
    assert n == sum((c + 31) // 32 for c in layout[:, 0])
    assert all(t[2] <= 32 and t[3] == (1 if t[2] >= 2 else 0) for t in tiles[:n])
    assert not tiles[n:].any()
    with pytest.raises(ValueError):
        O.expert_layout(np.array([7], np.uint32), 6, 4)


def test_add_rms():
    a, b = standard_x(64).reshape(2, 32), standard_x(64)[::-1].copy().reshape(2, 32)
    w = np.linspace(0.5, 1.5, 32, dtype=np.float32)
    s, y = O.add_rms(a, b, w, 1e-6)
    ss = a + b
    assert np.array_equal(s, ss)
    assert np.allclose(y, ss / np.sqrt((ss * ss).mean(-1, keepdims=True) + 1e-6) * w, rtol=1e-6)
