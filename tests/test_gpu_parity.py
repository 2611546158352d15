"""GPU parity: every operator of the path, through the C ABI, against the oracle
on the same seeded inputs, the committed golden vectors and the reference's own
synthetic fixtures.  Integer/byte work (dequantisation, routing ids, grouping) is
bit-exact; floating-point GEMV outputs are held to the reference's bound
|a - e| <= 1e-4 + 5e-5 |e| against an f64 dot of the dequantised weights."""
import glob
import os

import numpy as np
import pytest

from conftest import (lcg_q4k_fixture, q4_0_hand_expected, q4_0_hand_fixture, standard_x, tol_contract, tol_ref,
                      tol_ref_scaled)
from ingot_b200 import (BF16, F16, F32, Q4_0, Q4_K, Q6_K, Q8_0, InvalidData, Matrix, Tensor, Weight, synth)
from ingot_b200 import _abi
from oracle import oracle as O

pytestmark = pytest.mark.gpu

GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "decode_kind*.npz")))
QUANT = [Q4_K, Q6_K, Q4_0, Q8_0]


# ---- dequantisation: bit-exact ----------------------------------------------

@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p) for p in GOLDEN])
def test_dequant_matches_reference_golden_bits(gpu, path):
    g = np.load(path)
    m = Matrix.of(g["raw"], int(g["cols"]), int(g["rows"]), int(g["kind"]))
    got = gpu.dequant(m)
    assert np.array_equal(got.view(np.uint32), g["expected_bits"].reshape(-1))


@pytest.mark.parametrize("kind", [F32, F16, BF16] + QUANT)
def test_dequant_bit_exact_with_experts_and_tails(gpu, kind):
    for cols, rows, count in ((256, 1, 1), (512, 3, 2), (2560, 37, 3), (4096, 64, 1)):
        raw = synth.random_matrix(kind, cols, rows, count, seed=cols + kind)
        got = gpu.dequant(Matrix.of(raw, cols, rows, kind, count)).reshape(rows * count, cols)
        want = O.dequant(raw, cols, rows * count, kind)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (kind, cols, rows, count)


def test_dequant_config1_full_size_bit_exact(gpu):
    # configuration 1: W 4096x4096 Q4_K, seed 0; every one of the 16.7M weights
    raw = synth.random_matrix(Q4_K, 4096, 4096, seed=0)
    got = gpu.dequant(Matrix.of(raw, 4096, 4096, Q4_K)).reshape(4096, 4096)
    want = O.dequant(raw, 4096, 4096, Q4_K)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_dequant_unaligned_view_uses_scalar_path(gpu):
    raw = synth.random_matrix(Q6_K, 512, 5, seed=3)
    buf = gpu.bytes(np.concatenate([np.zeros(2, np.uint8), raw]))
    out = gpu.output(512 * 5)
    gpu.op(None, "read_rows", [buf.view_bytes(2, raw.size), out], [512, 5, 420, Q6_K])
    got = gpu.finish(None, out).reshape(5, 512)
    assert np.array_equal(got.view(np.uint32), O.dequant(raw, 512, 5, Q6_K).view(np.uint32))


def test_invalid_matrix_layouts_are_rejected(gpu):
    raw = synth.random_matrix(Q4_K, 512, 2, seed=0)
    with pytest.raises(InvalidData):
        gpu.dequant(Matrix(raw, 512, 2, 1, Q4_K, 144))            # wrong stride
    with pytest.raises(InvalidData):
        gpu.dequant(Matrix(raw[:-1], 512, 2, 1, Q4_K, 288))       # short data
    with pytest.raises(InvalidData):
        gpu.dequant(Matrix(raw, 512, 2, 1, 13, 288))              # Q5_K: outside this path
    with pytest.raises(InvalidData):
        gpu.project(Matrix.of(raw, 512, 2, Q4_K), np.zeros(511, np.float32))
    x = np.zeros(512, np.float32)
    x[3] = np.nan
    with pytest.raises(InvalidData):
        gpu.project(Matrix.of(raw, 512, 2, Q4_K), x)
    with pytest.raises(InvalidData):
        gpu.project(Matrix.of(synth.random_matrix(Q4_K, 512, 2, 2), 512, 2, Q4_K, 2), np.zeros(512, np.float32))


# ---- GEMV ----------------------------------------------------------------------

def gemv(gpu, raw, cols, rows, kind, x, expert=0, count_experts=1, x_kind=F32, plain=False, mma=True):
    x = np.ascontiguousarray(x, np.float32).reshape(-1, cols)
    w = gpu.bytes(raw)
    xb = gpu.floats(x) if x_kind == F32 else gpu.bf16(x)
    gpu.set_option(_abi.OPT_FORCE_PLAIN, int(plain))
    gpu.set_option(_abi.OPT_NO_MMA, int(not mma))
    try:
        y = gpu.matmul(None, w, cols, rows, synth.stride_of(kind, cols), kind, expert, xb, x.shape[0], x_kind)
        return gpu.finish(None, y).reshape(x.shape[0], rows)
    finally:
        gpu.set_option(_abi.OPT_FORCE_PLAIN, 0)
        gpu.set_option(_abi.OPT_NO_MMA, 0)


def test_config1_q4k_matvec(gpu):
    # configuration 1: 4096x4096 Q4_K, x ~ N(0,1) fp32, seed 0
    raw = synth.random_matrix(Q4_K, 4096, 4096, seed=0)
    x = synth.activations(1, 4096, seed=0)
    y = gemv(gpu, raw, 4096, 4096, Q4_K, x)
    e = O.matvec_f64(raw, 4096, 4096, Q4_K, x)
    err = np.abs(y - e)
    assert (err <= tol_contract(e)).all()
    assert (err <= tol_ref_scaled(e)).all(), float(err.max())      # the reference's tighter relative bound
    # with activations of model-like magnitude (outputs O(1)) the reference's bound holds as written
    xs = x * np.float32(1.0 / 256)
    ys, es = gemv(gpu, raw, 4096, 4096, Q4_K, xs), O.matvec_f64(raw, 4096, 4096, Q4_K, xs)
    assert (np.abs(ys - es) <= tol_ref(es)).all(), float(np.abs(ys - es).max())


SHAPES = {Q4_K: [(4096, 4096), (4096, 1024), (2560, 37), (768, 2048), (2048, 768), (256, 7), (12288, 33)],
          Q6_K: [(4096, 1024), (12288, 65), (2048, 5), (256, 3), (2560, 37)],
          Q4_0: [(2560, 2048), (10240, 33), (2048, 2560), (64, 7), (32, 1)],
          Q8_0: [(4096, 128), (2560, 37), (1024, 5), (32, 3)]}


@pytest.mark.parametrize("kind", QUANT)
@pytest.mark.parametrize("path", ["mma", "fp32", "plain"])
def test_gemv_matches_oracle(gpu, kind, path):
    plain = path == "plain"
    for cols, rows in SHAPES[kind]:
        raw = synth.random_matrix(kind, cols, rows, seed=rows)
        x = synth.activations(1, cols, seed=1)
        y = gemv(gpu, raw, cols, rows, kind, x, plain=plain, mma=path == "mma")
        e = O.matvec_f64(raw, cols, rows, kind, x)
        # the plain kernel sums 32 long lane-strided chains: held to the stated contract, not the tighter bound
        tol = tol_contract(e) if plain else tol_ref_scaled(e)
        assert (np.abs(y - e) <= tol).all(), (kind, cols, rows, float(np.abs(y - e).max()))


@pytest.mark.parametrize("kind", [F32, F16, BF16])
def test_float_weight_gemv(gpu, kind):
    for cols, rows in ((2048, 128), (32, 33), (100, 7)):
        raw = synth.random_matrix(kind, cols, rows, seed=5)
        x = synth.activations(3, cols, seed=2)
        y = gemv(gpu, raw, cols, rows, kind, x)
        e = O.matvec_f64(raw, cols, rows, kind, x)
        assert (np.abs(y - e) <= tol_ref(e)).all()


def test_f32_matmul_tails_and_expert_offsets(gpu):
    # src/metal/tests.rs:13-34
    for rows in (1, 3, 4, 5, 7, 33):
        raw = np.array([i // 32 + 1 for i in range(2 * rows * 32)], np.float32)
        w = gpu.floats(raw)
        for count in (1, 2, 4, 5, 8):
            x = gpu.floats(np.array([i // 32 + 1 for i in range(32 * count)], np.float32))
            y = gpu.finish(None, gpu.matmul(None, w, 32, rows, 128, F32, 1, x, count))
            exp = np.array([(rows + i % rows + 1) * 32 * (i // rows + 1) for i in range(rows * count)], float)
            assert np.abs(y - exp).max() < 2e-5


@pytest.mark.parametrize("mma", [False, True], ids=["fp32 kernels", "default path"])
@pytest.mark.parametrize("kind,cols", [(Q4_K, 2560), (Q6_K, 4096), (Q4_0, 2560), (Q8_0, 1024), (Q4_K, 12288)])
def test_token_counts_agree_bitwise_and_with_oracle(gpu, kind, cols, mma):
    # counts 2..8 bitwise equal to count 1 (src/expert_bench.rs:698-712) and tails of tokens: within the fp32
    # streaming kernels, and on the default path (one token: the int8 tensor-core kernel; 2..4: the same kernel
    # over a tile of rows; more than four tokens take the tensor-core GEMM there, as in the reference)
    rows = 37
    raw = synth.random_matrix(kind, cols, rows, seed=4)
    x = synth.activations(8, cols, seed=5)
    singles = np.concatenate([gemv(gpu, raw, cols, rows, kind, x[t], mma=mma) for t in range(8)])
    for n in ((2, 3, 4) if mma else (2, 3, 4, 5, 7, 8)):
        y = gemv(gpu, raw, cols, rows, kind, x[:n], mma=mma)
        assert np.array_equal(y.view(np.uint32), singles[:n].view(np.uint32)), (kind, n)
    e = O.matvec_f64(raw, cols, rows, kind, x)
    assert (np.abs(singles - e) <= tol_ref(e)).all()


@pytest.mark.parametrize("kind,cols,rows", [(Q4_K, 4096, 77), (Q6_K, 4096, 50), (Q4_0, 2560, 33), (Q8_0, 1024, 19)])
def test_packed_and_plain_activation_rows_meet_the_oracle(gpu, kind, cols, rows):
    from ingot_b200 import X_PACKED
    raw = synth.random_matrix(kind, cols, rows, seed=11)
    x = synth.activations(1, cols, seed=12)
    x[0, 5] = 70000.0                     # beyond binary16: exercises the power-of-two pre-scale
    w, xb = gpu.bytes(raw), gpu.floats(x)
    auto = gpu.finish(None, gpu.matmul(None, w, cols, rows, synth.stride_of(kind, cols), kind, 0, xb, 1))
    packed = gpu.pack_x(xb, 1, cols)
    y = gpu.finish(None, gpu.matmul(None, w, cols, rows, synth.stride_of(kind, cols), kind, 0, packed, 1, X_PACKED))
    # rows packed beforehand are binary16 with one scale per row; plain float32 rows become fixed point inside the
    # kernel with one scale per 32 columns, which the outlier cannot coarsen: both meet the oracle, the second tighter
    e = O.matvec_f64(raw, cols, rows, kind, x)[0]
    assert (np.abs(y - e) <= tol_contract(e)).all()
    assert (np.abs(auto - e) <= tol_ref_scaled(e)).all(), float(np.abs(auto - e).max())
    with pytest.raises(InvalidData):       # packed rows carry one token
        gpu.matmul(None, w, cols, rows, synth.stride_of(kind, cols), kind, 0, packed, 2, X_PACKED)


def test_expert_offset_and_lcg_fixture(gpu):
    # src/expert_bench.rs:648-749: LCG seed 23 blocks, cols 2560, rows 37, experts 3, expert 1
    data = lcg_q4k_fixture()
    x = standard_x(2560 * 4).reshape(4, 2560)
    y = gemv(gpu, data, 2560, 37, Q4_K, x, expert=1)
    e = O.matvec_f64(data, 2560, 37, Q4_K, x, expert=1)
    assert (np.abs(y - e) <= tol_ref(e)).all()
    w = gpu.dequant(Matrix.of(data, 2560, 37, Q4_K, 3)).reshape(3 * 37, 2560)
    assert np.array_equal(w.view(np.uint32), O.dequant(data, 2560, 3 * 37, Q4_K).view(np.uint32))


@pytest.mark.parametrize("kind", [Q4_K, Q6_K])
def test_bf16_activations(gpu, kind):
    cols, rows = 4096, 130
    raw = synth.random_matrix(kind, cols, rows, seed=8)
    x = synth.activations(2, cols, seed=9)
    xr = synth.from_bf16_bits(synth.to_bf16_bits(x))            # the oracle sees the same rounded x
    y = gemv(gpu, raw, cols, rows, kind, x, x_kind=BF16)
    e = O.matvec_f64(raw, cols, rows, kind, xr)
    assert (np.abs(y - e) <= tol_ref(e)).all()
    yp = gemv(gpu, raw, cols, rows, kind, x, x_kind=BF16, plain=True)
    assert (np.abs(yp - e) <= tol_contract(e)).all()


def test_project_host_and_weight_project(gpu):
    raw = synth.random_matrix(Q6_K, 4096, 77, seed=2)
    x = standard_x(4096)
    e = O.matvec_f64(raw, 4096, 77, Q6_K, x)[0]
    y = gpu.project(Matrix.of(raw, 4096, 77, Q6_K), x)
    assert (np.abs(y - e) <= tol_ref(e)).all()
    w = Weight.load(gpu, raw, [4096, 77], Q6_K)
    y2 = gpu.finish(None, w.project(gpu, gpu.command(), gpu.floats(x)))
    assert np.array_equal(y2.view(np.uint32), y.view(np.uint32))
    with pytest.raises(InvalidData):
        Weight.load(gpu, raw, [4096, 77], Q6_K, expect=[4096, 78])
    with pytest.raises(InvalidData):
        gpu.load_weight(raw[:-1], Tensor.of([4096, 77], Q6_K))


# ---- fused gate/up ---------------------------------------------------------------

@pytest.mark.parametrize("kind,cols,rows", [(Q4_K, 4096, 300), (Q4_0, 2560, 77), (Q6_K, 4096, 33), (Q8_0, 1024, 9)])
@pytest.mark.parametrize("gelu", [False, True], ids=["silu", "gelu"])
def test_gate_up_fused_equals_separate_and_oracle(gpu, kind, cols, rows, gelu):
    g, u = synth.random_matrix(kind, cols, rows, seed=1), synth.random_matrix(kind, cols, rows, seed=2)
    # scale inputs so the GLU is not saturated everywhere
    x = synth.activations(3, cols, seed=3) * np.float32(0.02 if kind in (Q4_K,) else 0.2)
    t = Tensor.of([cols, rows], kind)
    wg, wu = Weight(gpu.bytes(g), t), Weight(gpu.bytes(u), t)
    xb = gpu.floats(x)
    fused = gpu.finish(None, gpu.generic_gate_up(None, [wg, wu], xb, 3, gelu)).reshape(3, rows)
    yg = gpu.generic_project(None, wg, xb, 3)
    yu = gpu.generic_project(None, wu, xb, 3)
    sep = gpu.finish(None, gpu.activation(None, yg, yu, 3 * rows, gelu)).reshape(3, rows)
    assert np.array_equal(fused.view(np.uint32), sep.view(np.uint32))      # src/metal/tests.rs fused_gate_up_matches_separate
    eg, eu = O.matvec_f64(g, cols, rows, kind, x), O.matvec_f64(u, cols, rows, kind, x)
    e = O.glu(eg.astype(np.float32), eu.astype(np.float32), gelu=gelu).astype(np.float64)
    assert (np.abs(fused - e) <= tol_contract(e)).all(), float(np.abs(fused - e).max())
    other = Weight(wu.buffer, Tensor.of([cols, rows + 1], kind)) if rows > 1 else None
    assert gpu.generic_gate_up(None, [wg, other], xb, 3, gelu) is None      # shape mismatch -> no kernel


# ---- routed ------------------------------------------------------------------------

@pytest.mark.parametrize("plain", [False, True], ids=["stream", "plain"])
def test_routed_q4_0_hand_fixture(gpu, plain):
    # src/metal/tests.rs:35-93: 7 rows x 64 cols x 5 experts, top 3, shared and per-pair inputs
    rows, cols, experts, top = 7, 64, 5, 3
    w = gpu.bytes(q4_0_hand_fixture(rows, cols, experts))
    gpu.set_option(_abi.OPT_FORCE_PLAIN, int(plain))
    try:
        for tokens in (1, 2, 3, 5, 8):
            pairs = tokens * top
            ids = np.array([(i * 7 + 1) % experts for i in range(pairs)], np.uint32)
            idb = gpu.bytes(ids)
            for per in (False, True):
                inputs = np.array([(i % 19) * 0.125 - 1.0 for i in range(cols * (pairs if per else tokens))], np.float32)
                y = gpu.output(rows * pairs)
                gpu.op(None, "project_routed_batch", [w, gpu.floats(inputs), idb, y], [cols, rows, 36, 2, top, int(per)],
                       rows, pairs)
                got = gpu.finish(None, y).reshape(pairs, rows)
                assert np.abs(got - q4_0_hand_expected(ids, rows, cols, top, per, inputs)).max() < 2e-5
    finally:
        gpu.set_option(_abi.OPT_FORCE_PLAIN, 0)


def test_routed_moe_shapes_match_oracle(gpu):
    # configuration 4 shapes: 128 experts, gate/up 2048->768, down 768->2048, Q4_K, top 8
    experts, hidden, ffn, top = 16, 2048, 768, 8          # 16 experts keep the upload small
    tg = Tensor.of([hidden, ffn, experts], Q4_K)
    td = Tensor.of([ffn, hidden, experts], Q4_K)
    g, u = synth.random_matrix(Q4_K, hidden, ffn, experts, 1), synth.random_matrix(Q4_K, hidden, ffn, experts, 2)
    d = synth.random_matrix(Q4_K, ffn, hidden, experts, 3)
    wg, wu, wd = Weight(gpu.bytes(g), tg), Weight(gpu.bytes(u), tg), Weight(gpu.bytes(d), td)
    for tokens in (1, 4):
        pairs = tokens * top
        rng = np.random.default_rng(tokens)
        ids = np.stack([rng.permutation(experts)[:top] for _ in range(tokens)]).astype(np.uint32).reshape(-1)
        x = synth.activations(tokens, hidden, seed=7) * np.float32(0.01)
        idb, xb = gpu.bytes(ids), gpu.floats(x)
        act_b = gpu.generic_routed_gate_up(None, [wg, wu], [xb, idb], top, pairs)
        act = gpu.finish(None, act_b).reshape(pairs, ffn)
        out_b = gpu.output(pairs * hidden)
        assert gpu.generic_routed(None, wd, [act_b, idb, out_b], True, top, pairs)
        out = gpu.finish(None, out_b).reshape(pairs, hidden)
        for p in range(pairs):
            e_id, t = int(ids[p]), p // top
            eg = O.matvec_f64(g, hidden, ffn, Q4_K, x[t], expert=e_id)[0]
            eu = O.matvec_f64(u, hidden, ffn, Q4_K, x[t], expert=e_id)[0]
            ea = O.glu(eg.astype(np.float32), eu.astype(np.float32)).astype(np.float64)
            assert (np.abs(act[p] - ea) <= tol_contract(ea)).all()
            ed = O.matvec_f64(d, ffn, hidden, Q4_K, act[p], expert=e_id)[0]     # same input as the GPU's down-proj
            assert (np.abs(out[p] - ed) <= tol_contract(ed)).all()
            assert (np.abs(out[p] - ed) <= tol_ref_scaled(ed)).all()


def test_routed_expert_id_out_of_range_is_an_error_not_a_fault(gpu):
    t = Tensor.of([256, 4, 2], Q4_K)
    w = Weight(gpu.bytes(synth.random_matrix(Q4_K, 256, 4, 2)), t)
    ids = gpu.bytes(np.array([0, 5], np.uint32))
    y = gpu.zeros(8)
    assert gpu.generic_routed(None, w, [gpu.floats(np.ones(256, np.float32)), ids, y], False, 2, 2)
    with pytest.raises(InvalidData, match="expert id out of range"):
        gpu.complete()
    # the handle stays usable and the valid pair was computed
    gpu.complete()
    assert np.isfinite(gpu.read_f32(y)).all()


# ---- routing, combine, grouping ---------------------------------------------------

@pytest.mark.parametrize("count", [1, 31, 33, 128, 288, 512])
@pytest.mark.parametrize("ties", [False, True])
def test_route_topk_ids_exact_weights_close(gpu, count, ties):
    # src/metal/tests.rs:94-137
    logits = np.array([1000.0 if ties else float((i * 17) % 23) - 11.0 for i in range(count)], np.float32)
    top = min(count, 10)
    ids_b, w_b = gpu.route_topk(gpu.floats(logits), count, top, 1)
    gpu.complete()
    e_ids, e_w = O.route(logits, top)
    assert gpu.read_u32(ids_b, top).tolist() == e_ids.tolist()
    assert np.abs(gpu.read_f32(w_b, top) - e_w).max() < 2e-5


def test_route_topk_batch_of_random_tokens(gpu):
    # configuration 4: 128 experts, N(0,1) logits, top-8 softmax renormalised, 32 tokens
    logits = np.random.default_rng(0).normal(0, 1, (32, 128)).astype(np.float32)
    ids_b, w_b = gpu.route_topk(gpu.floats(logits), 128, 8, 32)
    gpu.complete()
    ids, w = gpu.read_u32(ids_b, 256).reshape(32, 8), gpu.read_f32(w_b, 256).reshape(32, 8)
    for t in range(32):
        e_ids, e_w = O.route(logits[t], 8)
        assert ids[t].tolist() == e_ids.tolist()
        assert np.abs(w[t] - e_w).max() < 2e-6
    assert np.abs(w.sum(1) - 1).max() < 1e-6


def test_route_rejects_bad_requests(gpu):
    l = gpu.floats(np.zeros(8, np.float32))
    for experts, top in ((8, 0), (8, 9), (1024, 4)):
        with pytest.raises(InvalidData):
            gpu.route_topk(l, experts, top, 1)
    bad = gpu.floats(np.array([0.0, np.nan, 1.0, 2.0], np.float32))
    gpu.route_topk(bad, 4, 2, 1)
    with pytest.raises(InvalidData, match="invalid router scores"):
        gpu.complete()
    gpu.complete()


def test_moe_sum_and_merge(gpu):
    rng = np.random.default_rng(3)
    tokens, top, width = 5, 8, 2048
    routed = rng.normal(0, 1, (tokens * top, width)).astype(np.float32)
    w = rng.random((tokens, top)).astype(np.float32)
    y = gpu.finish(None, gpu.moe_sum(gpu.floats(routed), gpu.floats(w), width, top, tokens)).reshape(tokens, width)
    assert np.abs(y - O.moe_sum(routed, w, width, top)).max() < 1e-5
    shared = rng.normal(0, 1, width).astype(np.float32)
    out = gpu.finish(None, gpu.merge(None, gpu.floats(routed[:top]), gpu.floats(shared), gpu.floats(w[0]),
                                     gpu.floats(np.array([0.3], np.float32)), width, top))
    assert np.abs(out - O.combine(routed[:top], shared, w[0], 0.3, width)).max() < 1e-5


def test_expert_layout_and_combine_packed(gpu):
    rng = np.random.default_rng(11)
    for pairs, experts in ((8, 128), (64, 128), (256, 128), (100, 6), (1, 1)):
        ids = rng.integers(0, experts, pairs).astype(np.uint32)
        cap = pairs + experts
        layout, tiles, packed, inverse = gpu.expert_layout(gpu.bytes(ids), pairs, experts, cap)
        gpu.complete()
        e_layout, e_tiles, e_pairs, e_inv, n = O.expert_layout(ids, experts, cap)
        assert np.array_equal(gpu.read_u32(layout, 2 * experts).reshape(-1, 2), e_layout)
        assert np.array_equal(gpu.read_u32(tiles, 4 * cap).reshape(-1, 4), e_tiles)
        assert np.array_equal(gpu.read_u32(packed, pairs), e_pairs)
        assert np.array_equal(gpu.read_u32(inverse, pairs), e_inv)
    top, tokens, width = 8, 8, 256
    ids = rng.integers(0, 16, top * tokens).astype(np.uint32)
    _, _, packed, inverse = gpu.expert_layout(gpu.bytes(ids), top * tokens, 16, 80)
    gpu.complete()
    inv = gpu.read_u32(inverse, top * tokens)
    routed_packed = rng.normal(0, 1, (top * tokens, width)).astype(np.float32)
    w = rng.random(top * tokens).astype(np.float32)
    y = gpu.finish(None, gpu.combine_packed(gpu.floats(routed_packed), gpu.floats(w), inverse, width, top, tokens))
    assert np.abs(y.reshape(tokens, width) - O.combine_packed(routed_packed, w, inv, width, top)).max() < 1e-5


def test_add_rms(gpu):
    rng = np.random.default_rng(1)
    a, b = rng.normal(0, 1, (3, 4096)).astype(np.float32), rng.normal(0, 1, (3, 4096)).astype(np.float32)
    w = rng.random(4096).astype(np.float32) + 0.5
    s_b, y_b, yb_b = gpu.add_rms(None, gpu.floats(a), gpu.floats(b), gpu.floats(w), 4096, 3, 1e-6, True, bf16_out=True)
    y = gpu.finish(None, y_b).reshape(3, 4096)
    e_s, e_y = O.add_rms(a, b, w, 1e-6)
    assert np.array_equal(gpu.read_f32(s_b).reshape(3, 4096), e_s)
    assert np.abs(y - e_y).max() < 1e-5
    assert np.array_equal(gpu.read_bytes(yb_b).view(np.uint16).reshape(3, 4096), synth.to_bf16_bits(y))


def test_add_rms_packed_equals_separate_pack(gpu):
    import ctypes as C
    rng = np.random.default_rng(4)
    a, b = rng.normal(0, 1, (1, 4096)).astype(np.float32), rng.normal(0, 1, (1, 4096)).astype(np.float32)
    ab, bb = gpu.floats(a), gpu.floats(b)
    n = gpu.packed_x_bytes(4096)
    for from_bf16 in (0, 1):
        s, y, y16, fused = gpu.output(4096), gpu.output(4096), gpu.empty_bytes(2 * 4096), gpu.empty_bytes(n)
        gpu._check(gpu._lib.ingot_add_rms_packed(gpu._h, ab.ptr, bb.ptr, None, s.ptr, y.ptr, y16.ptr, fused.ptr, from_bf16,
                                                 4096, 1, 1e-6, 1))
        separate = gpu.pack_x(y16 if from_bf16 else y, 1, 4096, BF16 if from_bf16 else F32)
        gpu.complete()
        assert np.array_equal(gpu.read_bytes(fused)[:n - 12], gpu.read_bytes(separate)[:n - 12])    # the tail pads to 16 bytes


# ---- recorded commands ---------------------------------------------------------------

def test_recorded_chain_replays_identically(gpu):
    # a small q -> o style chain recorded once (one Command per decode step) and replayed
    cols = 1024
    w1 = Weight(gpu.bytes(synth.random_matrix(Q4_K, cols, cols, seed=1)), Tensor.of([cols, cols], Q4_K))
    w2 = Weight(gpu.bytes(synth.random_matrix(Q6_K, cols, 256, seed=2)), Tensor.of([cols, 256], Q6_K))
    x = gpu.floats(synth.activations(1, cols, seed=3))
    h, n, y = gpu.output(cols), gpu.output(cols), gpu.output(256)
    def chain():
        gpu.matmul(None, w1.buffer, cols, cols, w1.t.stride, Q4_K, 0, x, 1, out=h)
        gpu._check(gpu._lib.ingot_add_rms(gpu._h, h.ptr, None, None, None, n.ptr, None, cols, 1, 1e-6, 0))
        gpu.matmul(None, w2.buffer, cols, 256, w2.t.stride, Q6_K, 0, n, 1, out=y)
    chain()
    eager = gpu.finish(None, y).copy()
    gpu.record()
    chain()
    graph = gpu.end_record()
    for _ in range(3):
        gpu._check(gpu._lib.ingot_buffer_zero(gpu._h, y.ptr, y.nbytes))
        graph.submit()
        assert np.array_equal(gpu.finish(None, y).view(np.uint32), eager.view(np.uint32))


# ---- MoE layer and its expert-parallel split -------------------------------------------

def test_moe_layer_matches_oracle_and_expert_shards_sum_to_it(gpu):
    from ingot_b200.moe import MoeChain, MoeShape
    shape = MoeShape("test", 1, 512, 16, 4, 256, Q4_K)
    tokens = 3
    rng = np.random.default_rng(7)
    logits = rng.normal(0, 1, (tokens, shape.experts)).astype(np.float32)
    x = synth.activations(tokens, shape.hidden, seed=8) * np.float32(0.02)

    def run(rank, world):
        c = MoeChain(gpu, shape, tokens=tokens, seed=3, rank=rank, world=world, all_reduce=lambda buf, n: None,
                     keep_host=True)
        gpu._check(gpu._lib.ingot_buffer_upload(gpu._h, c.logits.ptr, logits.ctypes.data, logits.nbytes))
        gpu._check(gpu._lib.ingot_buffer_upload(gpu._h, c.x.ptr, x.ctypes.data, x.nbytes))
        c.layer(0)
        return gpu.finish(None, c.y).reshape(tokens, shape.hidden).copy(), c

    full, chain = run(0, 1)
    ws = chain.weights[0]
    e = np.zeros((tokens, shape.hidden))
    for t in range(tokens):
        ids, w = O.route(logits[t], shape.top)
        for k, wt in zip(ids, w):
            a = O.glu(O.matvec_f64(ws["gate_host"], 512, 256, Q4_K, x[t], expert=int(k))[0].astype(np.float32),
                      O.matvec_f64(ws["up_host"], 512, 256, Q4_K, x[t], expert=int(k))[0].astype(np.float32))
            e[t] += float(wt) * O.matvec_f64(ws["down_host"], 256, 512, Q4_K, a, expert=int(k))[0]
    assert (np.abs(full - e) <= tol_contract(e)).all(), float(np.abs(full - e).max())
    parts = sum(run(r, 4)[0].astype(np.float64) for r in range(4))       # four expert shards, one after the other
    assert np.abs(parts - full).max() <= 1e-5 * max(1.0, float(np.abs(full).max()))


# ---- prefill GEMM on the tensor cores ------------------------------------------------------

@pytest.mark.parametrize("kind", [Q4_K, Q6_K, Q4_0])
@pytest.mark.parametrize("cols,rows,tokens", [(256, 128, 16), (512, 200, 70), (1024, 128, 256), (2560, 37, 32), (4096, 300, 513),
                                              (512, 128, 300), (768, 140, 600)])
def test_gemm_matches_f16_staged_expectation(gpu, kind, cols, rows, tokens):
    # src/expert_bench.rs:734-749: wide GEMM against an f64 dot of F16-rounded weights (and activations)
    raw = synth.random_matrix(kind, cols, rows, 2, seed=cols + rows)
    x = standard_x(cols * tokens).reshape(tokens, cols)             # multiples of 1/32: exact in binary16
    w, xb = gpu.bytes(raw), gpu.floats(x)
    y = gpu.finish(None, gpu.gemm(None, w, cols, rows, synth.stride_of(kind, cols), kind, 1, xb, tokens)).reshape(tokens, rows)
    e = O.gemm_f16_f64(raw, cols, rows, kind, x, expert=1)
    assert (np.abs(y - e) <= tol_ref_scaled(e)).all(), float(np.abs(y - e).max())
    # the same through Gpu::matmul, which takes the GEMM for more than four tokens, and with bf16 activations
    if tokens > 4:
        y2 = gpu.finish(None, gpu.matmul(None, w, cols, rows, synth.stride_of(kind, cols), kind, 1, xb, tokens))
        assert np.array_equal(y2.view(np.uint32), y.reshape(-1).view(np.uint32))
        y3 = gpu.finish(None, gpu.gemm(None, w, cols, rows, synth.stride_of(kind, cols), kind, 1, gpu.bf16(x), tokens, BF16))
        assert np.array_equal(y3.view(np.uint32), y.reshape(-1).view(np.uint32))      # these x are exact in bf16 too


def test_gemm_random_activations_and_unsupported_shapes(gpu):
    cols, rows, tokens = 2048, 256, 130
    raw = synth.random_matrix(Q4_K, cols, rows, seed=3)
    x = synth.activations(tokens, cols, seed=4)
    w, xb = gpu.bytes(raw), gpu.floats(x)
    y = gpu.finish(None, gpu.gemm(None, w, cols, rows, synth.stride_of(Q4_K, cols), Q4_K, 0, xb, tokens)).reshape(tokens, rows)
    e = O.gemm_f16_f64(raw, cols, rows, Q4_K, x)
    assert (np.abs(y - e) <= tol_ref_scaled(e)).all(), float(np.abs(y - e).max())
    exact = O.matvec_f64(raw, cols, rows, Q4_K, x)
    assert np.abs(y - exact).max() <= 2e-3 * np.abs(exact).max()                       # F16 staging: ~1e-3 of full precision
    with pytest.raises(InvalidData):
        gpu.gemm(None, w, cols, rows, synth.stride_of(Q4_K, cols), Q6_K, 0, xb, tokens)          # layout mismatch
    w0 = gpu.bytes(synth.random_matrix(Q8_0, 256, 8, seed=1))
    with pytest.raises(InvalidData):
        gpu.gemm(None, w0, 256, 8, synth.stride_of(Q8_0, 256), Q8_0, 0, xb, 8)                   # no tensor-core kernel


# ---- one-token GEMV on the tcgen05 int8 tensor cores -----------------------------------------

def _tc_gemv(gpu, raw, cols, rows, x, x_kind=F32, expert=0):
    w = gpu.bytes(raw)
    xb = gpu.floats(x) if x_kind == F32 else gpu.bf16(x)
    gpu.set_option(_abi.OPT_TCGEN05_GEMV, 1)
    try:
        return gpu.finish(None, gpu.matmul(None, w, cols, rows, synth.stride_of(Q4_K, cols), Q4_K, expert, xb, 1, x_kind))
    finally:
        gpu.set_option(_abi.OPT_TCGEN05_GEMV, 0)


@pytest.mark.parametrize("cols,rows", [(256, 128), (512, 100), (4096, 300), (2560, 37), (4096, 4096), (12288, 256)])
def test_tcgen05_gemv_q4k_matches_oracle(gpu, cols, rows):
    raw = synth.random_matrix(Q4_K, cols, rows, 2, seed=cols + rows)
    x = synth.activations(1, cols, seed=5) / 256.0
    y = _tc_gemv(gpu, raw, cols, rows, x, expert=1)
    e = O.matvec_f64(raw, cols, rows, Q4_K, x, expert=1)[0]
    assert (np.abs(y - e) <= tol_ref(e)).all(), float(np.abs(y - e).max())
    # run to run the result is the same bits (the tile sums do not depend on arrival order)
    y2 = _tc_gemv(gpu, raw, cols, rows, x, expert=1)
    assert np.array_equal(y.view(np.uint32), y2.view(np.uint32))


# ---- independent projections ---------------------------------------------------------------

def test_independent_scope_matches_serial_issue_and_records(gpu):
    # q, k, v style: three projections of the same packed activations, issued concurrently
    from ingot_b200 import X_PACKED
    cols = 4096
    shapes = [(Q4_K, 512), (Q4_K, 128), (Q6_K, 128)]
    raws = [synth.random_matrix(k, cols, r, seed=60 + i) for i, (k, r) in enumerate(shapes)]
    ws = [gpu.bytes(r) for r in raws]
    x = synth.activations(1, cols, seed=61) / 256.0
    packed = gpu.pack_x(gpu.floats(x), 1, cols)

    def issue():
        return [gpu.matmul(None, w, cols, r, synth.stride_of(k, cols), k, 0, packed, 1, X_PACKED) for w, (k, r) in zip(ws, shapes)]

    serial = [gpu.finish(None, y) for y in issue()]
    with gpu.independent():
        ys = issue()
    par = [gpu.finish(None, y) for y in ys]
    for a, b, raw, (k, r) in zip(serial, par, raws, shapes):
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
        e = O.matvec_f64(raw, cols, r, k, x)[0]
        assert (np.abs(b - e) <= tol_ref(e)).all()
    # inside a recorded command, replayed twice
    outs = [gpu.output(r) for _, r in shapes]
    gpu.record()
    with gpu.independent():
        for w, (k, r), y in zip(ws, shapes, outs):
            gpu._check(gpu._lib.ingot_matmul(gpu._h, w.ptr, cols, r, synth.stride_of(k, cols), k, 0, packed.ptr, X_PACKED, 1, y.ptr))
    graph = gpu.end_record()
    for _ in range(2):
        for y in outs:
            gpu._check(gpu._lib.ingot_buffer_zero(gpu._h, y.ptr, y.nbytes))
        graph.submit()
        gpu.complete()
        for a, y in zip(serial, outs):
            assert np.array_equal(a.view(np.uint32), gpu.read_f32(y).view(np.uint32))
    with pytest.raises(InvalidData):          # a scope cannot be left open at the end of a recording, nor nested
        with gpu.independent():
            with gpu.independent():
                pass


def test_independent_scope_groups_mixed_types_and_shapes(gpu):
    # five projections, four weight types, two activation widths: the scope launches them as
    # grids of up to four parts; every part must equal the same call issued alone
    from ingot_b200 import X_PACKED
    parts = [(Q4_K, 4096, 520), (Q6_K, 4096, 136), (Q4_0, 2560, 77), (Q8_0, 2560, 40), (Q4_K, 4096, 16)]
    raws = [synth.random_matrix(k, c, r, seed=160 + i) for i, (k, c, r) in enumerate(parts)]
    ws = [gpu.bytes(r) for r in raws]
    xs = {c: synth.activations(1, c, seed=170 + c) / 128.0 for c in (4096, 2560)}
    packed = {c: gpu.pack_x(gpu.floats(x), 1, c) for c, x in xs.items()}

    def issue():
        return [gpu.matmul(None, w, c, r, synth.stride_of(k, c), k, 0, packed[c], 1, X_PACKED) for w, (k, c, r) in zip(ws, parts)]

    alone = [gpu.finish(None, y) for y in issue()]
    with gpu.independent():
        ys = issue()
    grouped = [gpu.finish(None, y) for y in ys]
    for a, b, raw, (k, c, r) in zip(alone, grouped, raws, parts):
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
        e = O.matvec_f64(raw, c, r, k, xs[c])[0]
        assert (np.abs(b - e) <= tol_ref(e)).all()


# ---- add_rms fused into the projection ------------------------------------------------------

@pytest.mark.parametrize("kind,cols,rows", [(Q4_K, 4096, 300), (Q6_K, 4096, 130), (Q4_0, 2560, 77), (Q4_K, 12288, 64)])
@pytest.mark.parametrize("add,bf16", [(0, 0), (1, 1)])
def test_normed_projection_matches_add_rms_then_matmul(gpu, kind, cols, rows, add, bf16):
    from ingot_b200 import X_PACKED
    raw = synth.random_matrix(kind, cols, rows, seed=71)
    rng = np.random.default_rng(72)
    a, b = rng.normal(0, 3, (1, cols)).astype(np.float32), rng.normal(0, 1, (1, cols)).astype(np.float32)
    w, ab, bb = gpu.bytes(raw), gpu.floats(a), gpu.floats(b)
    stride = synth.stride_of(kind, cols)
    s_f, y_f = gpu.output(cols), gpu.output(rows)
    gpu._check(gpu._lib.ingot_matmul_normed(gpu._h, w.ptr, cols, rows, stride, kind, 0, ab.ptr, bb.ptr, None, s_f.ptr, 1e-6, add, bf16, y_f.ptr))
    fused = gpu.finish(None, y_f)
    # separately: add_rms with a packed output, then the projection
    s_s, packed = gpu.output(cols), gpu.empty_bytes(gpu.packed_x_bytes(cols))
    gpu._check(gpu._lib.ingot_add_rms_packed(gpu._h, ab.ptr, bb.ptr, None, s_s.ptr, None, None, packed.ptr, bf16, cols, 1, 1e-6, add))
    sep = gpu.finish(None, gpu.matmul(None, w, cols, rows, stride, kind, 0, packed, 1, X_PACKED))
    # the reference's bound against an f64 dot of the normalised (and bfloat16-rounded) row, plus, with bfloat16
    # rounding, what the columns whose rounding hangs on the last float32 bits of the norm can move (one bfloat16
    # step each: oracle/chain_check.py).  The separate path differs from the fused one by the order of the sum of
    # squares and by its activation row form (binary16 parts against fixed point): each meets the bound by itself.
    from oracle.chain_check import expect_projection
    _, e, tol = expect_projection(raw, cols, rows, kind, a[0], b[0] if add else None, bool(bf16))
    assert (np.abs(fused - e) <= tol).all(), float((np.abs(fused - e) / tol).max())
    assert (np.abs(sep - e) <= tol).all(), float((np.abs(sep - e) / tol).max())
    if add:
        assert np.array_equal(gpu.read_f32(s_f).view(np.uint32), gpu.read_f32(s_s).view(np.uint32))
        with pytest.raises(InvalidData):        # the sum cannot go over an input
            gpu._check(gpu._lib.ingot_matmul_normed(gpu._h, w.ptr, cols, rows, stride, kind, 0, ab.ptr, bb.ptr, None, ab.ptr, 1e-6, 1, bf16, y_f.ptr))


def test_fused_and_unfused_chains_agree(gpu):
    from ingot_b200.chain import QWEN3_8B, DecodeChain
    h0 = np.random.default_rng(1).normal(0, 1, (1, QWEN3_8B.hidden)).astype(np.float32)
    logits = []
    for fused in (False, True):
        chain = DecodeChain(gpu, QWEN3_8B, batch=1, x_kind=BF16, seed=3, layers=2, fused_norm=fused)
        gpu._check(gpu._lib.ingot_buffer_upload(gpu._h, chain.h_in.ptr, h0.ctypes.data, h0.nbytes))
        chain.step()
        gpu.complete()
        logits.append(gpu.read_f32(chain.logits))
        assert chain.fused_norm == fused
        del chain
    scale = float(np.sqrt(np.mean(np.square(logits[0]))))
    assert np.abs(logits[0] - logits[1]).max() <= 2e-2 * scale     # bfloat16 rounding points move with the sum order


def test_row_sharded_chain_matches_the_unsharded_chain(gpu):
    # two ranks of the row-sharded (tensor-parallel) step in lock step on one device, the all-gather done
    # through the host: every rank's logits equal the unsharded chain's bit for bit (a row's arithmetic
    # does not depend on which rank or CTA owns it)
    import threading
    from ingot_b200 import Gpu
    from ingot_b200.chain import QWEN3_8B, DecodeChain
    h0 = np.random.default_rng(1).normal(0, 1, (1, QWEN3_8B.hidden)).astype(np.float32)
    ref = DecodeChain(gpu, QWEN3_8B, batch=1, x_kind=BF16, seed=3, layers=2)
    gpu._check(gpu._lib.ingot_buffer_upload(gpu._h, ref.h_in.ptr, h0.ctypes.data, h0.nbytes))
    ref.step()
    gpu.complete()
    want = gpu.read_f32(ref.logits).copy()
    del ref
    world = 2
    handles = [Gpu(0) for _ in range(world)]
    slots, bar, errors, got = [None] * world, threading.Barrier(world, timeout=120), [], [None] * world

    def gather_for(r):
        def all_gather(part, full, batch, rows_local):
            g = handles[r]
            g.complete()
            slots[r] = g.read_f32(part, batch * rows_local).copy()
            bar.wait()
            whole = np.concatenate(slots)
            bar.wait()
            g._check(g._lib.ingot_buffer_upload(g._h, full.ptr, whole.ctypes.data, whole.nbytes))
        return all_gather

    def run(r):
        try:
            g = handles[r]
            c = DecodeChain(g, QWEN3_8B, batch=1, x_kind=BF16, seed=3, layers=2, rank=r, world=world, all_gather=gather_for(r))
            assert c.fused_norm
            g._check(g._lib.ingot_buffer_upload(g._h, c.h_in.ptr, h0.ctypes.data, h0.nbytes))
            c.step()
            g.complete()
            got[r] = g.read_f32(c.logits).copy()
        except Exception as e:          # a failed rank must not leave the other one waiting
            errors.append(e)
            bar.abort()

    threads = [threading.Thread(target=run, args=(r,)) for r in range(world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    for g in handles:
        g.close()
    assert not errors, errors
    for r in range(world):
        assert np.array_equal(got[r].view(np.uint32), want.view(np.uint32))


# ---- Gpu::moe (host-vector convenience) -------------------------------------------------------

def test_moe_host_wrapper_matches_oracle(gpu):
    # src/metal.rs:1663-1713: selected experts' FFNs + shared expert, merged with a sigmoid gate
    width, ffn, top = 512, 256, 4
    rng = np.random.default_rng(9)
    mk = lambda kind, cols, rows, count, seed: Matrix.of(synth.random_matrix(kind, cols, rows, count, seed=seed), cols, rows, kind, count)
    routed = [mk(Q4_K, width, ffn, top, 1), mk(Q4_K, width, ffn, top, 2), mk(Q4_K, ffn, width, top, 3)]
    shared = [mk(Q4_K, width, ffn, 1, 4), mk(Q4_K, width, ffn, 1, 5), mk(Q4_K, ffn, width, 1, 6)]
    gate = Matrix.of(rng.normal(0, 0.05, width).astype(np.float32).view(np.uint8), width, 1, F32)
    x = (rng.normal(0, 1, width) / 64).astype(np.float32)
    weights = np.array([0.4, 0.3, 0.2, 0.1], np.float32)
    y = gpu.moe(routed, shared, gate, x, weights)

    def expert_ffn(ms, e):
        g = O.matvec_f64(ms[0].data, width, ffn, Q4_K, x.reshape(1, -1), expert=e)[0]
        u = O.matvec_f64(ms[1].data, width, ffn, Q4_K, x.reshape(1, -1), expert=e)[0]
        act = O.glu(g.astype(np.float32), u.astype(np.float32))
        return O.matvec_f64(ms[2].data, ffn, width, Q4_K, act.reshape(1, -1), expert=e)[0]

    routed_e = np.stack([expert_ffn(routed, e) for e in range(top)]).astype(np.float32)
    shared_e = expert_ffn(shared, 0).astype(np.float32)
    logit = float(np.dot(gate.data.view(np.float32).astype(np.float64), x.astype(np.float64)))
    e = O.combine(routed_e, shared_e, weights, logit, width).astype(np.float64)
    # three chained projections: the bound of the last one plus the first two's carried through it would be the
    # principled figure; the layer's outputs are O(1e-3) here, so the reference's plain bound is checked instead
    assert (np.abs(y - e) <= tol_ref(e)).all(), float(np.abs(y - e).max())
    with pytest.raises(InvalidData):
        gpu.moe(routed, shared, gate, x, weights[:3])


def test_gate_up_wide_batch_takes_the_gemm(gpu):
    cols, rows, tokens = 1024, 300, 9
    g_raw, u_raw = synth.random_matrix(Q4_K, cols, rows, seed=81), synth.random_matrix(Q4_K, cols, rows, seed=82)
    x = standard_x(cols * tokens).reshape(tokens, cols) * np.float32(0.5)
    t = Tensor.of([cols, rows], Q4_K)
    wg, wu = Weight(gpu.bytes(g_raw), t), Weight(gpu.bytes(u_raw), t)
    y = gpu.finish(None, gpu.generic_gate_up(None, [wg, wu], gpu.floats(x), tokens, False)).reshape(tokens, rows)
    eg, eu = O.gemm_f16_f64(g_raw, cols, rows, Q4_K, x), O.gemm_f16_f64(u_raw, cols, rows, Q4_K, x)
    e = O.glu(eg.astype(np.float32), eu.astype(np.float32)).reshape(tokens, rows).astype(np.float64)
    # act = silu(g) u: the two GEMM bounds carried through the activation (|d act| <= 1.13 |u| dg + |silu(g)| du)
    tg, tu = tol_ref_scaled(eg.reshape(tokens, rows)), tol_ref_scaled(eu.reshape(tokens, rows))
    eg2, eu2 = eg.reshape(tokens, rows), eu.reshape(tokens, rows)
    silu = np.abs(eg2 / (1.0 + np.exp(-eg2)))
    tol = 1.13 * np.abs(eu2) * tg + (silu + 1.13 * tg) * tu + 4e-6 * np.abs(e) + 1e-30
    assert (np.abs(y - e) <= tol).all(), float((np.abs(y - e) / tol).max())


# ---- several tokens per pass over the weights (high-part rows) ---------------------------------

@pytest.mark.parametrize("kind,cols,rows", [(Q4_K, 4096, 300), (Q6_K, 4096, 130), (Q4_K, 2048, 16), (Q6_K, 12288, 40)])
@pytest.mark.parametrize("tokens", [1, 2, 5, 8, 11])
def test_multi_token_gemv_on_high_part_rows(gpu, kind, cols, rows, tokens):
    from ingot_b200 import X_PACKED_HI
    raw = synth.random_matrix(kind, cols, rows, 2, seed=91)
    x = synth.activations(tokens, cols, seed=92) / 256.0
    xr = synth.from_bf16_bits(synth.to_bf16_bits(x))
    w = gpu.bytes(raw)
    stride = synth.stride_of(kind, cols)
    packed = gpu.pack_x_hi(gpu.bf16(x), tokens, cols)
    y = gpu.finish(None, gpu.matmul(None, w, cols, rows, stride, kind, 1, packed, tokens, X_PACKED_HI)).reshape(tokens, rows)
    e = O.matvec_f64(raw, cols, rows, kind, xr, expert=1)
    assert (np.abs(y - e) <= tol_ref(e)).all(), float(np.abs(y - e).max())
    if tokens > 1:       # each token agrees with the one-token kernel on the same row to summation-order noise
        one = gpu.finish(None, gpu.matmul(None, w, cols, rows, stride, kind, 1, packed, 1, X_PACKED_HI))
        assert (np.abs(one - y[0]) <= 2 * tol_ref(e[0])).all()


def test_multi_token_gate_up_and_chain(gpu):
    from ingot_b200 import X_PACKED_HI
    from ingot_b200.chain import QWEN3_8B, DecodeChain
    cols, rows, tokens = 4096, 200, 8
    g_raw, u_raw = synth.random_matrix(Q4_K, cols, rows, seed=93), synth.random_matrix(Q4_K, cols, rows, seed=94)
    x = synth.activations(tokens, cols, seed=95) * np.float32(0.02)
    xr = synth.from_bf16_bits(synth.to_bf16_bits(x))
    packed = gpu.pack_x_hi(gpu.bf16(x), tokens, cols)
    y = gpu.output(tokens * rows)
    wg, wu = gpu.bytes(g_raw), gpu.bytes(u_raw)
    gpu._check(gpu._lib.ingot_gate_up(gpu._h, wg.ptr, wu.ptr, cols, rows, synth.stride_of(Q4_K, cols), Q4_K,
                                      packed.ptr, X_PACKED_HI, tokens, 0, y.ptr))
    got = gpu.finish(None, y).reshape(tokens, rows)
    eg, eu = O.matvec_f64(g_raw, cols, rows, Q4_K, xr), O.matvec_f64(u_raw, cols, rows, Q4_K, xr)
    e = O.glu(eg.astype(np.float32), eu.astype(np.float32)).reshape(tokens, rows).astype(np.float64)
    assert (np.abs(got - e) <= tol_contract(e)).all(), float(np.abs(got - e).max())
    # the batch-8 chain: every token's logits equal the batch-1 chain's on the same input, to bfloat16 noise
    h0 = np.random.default_rng(1).normal(0, 1, (8, QWEN3_8B.hidden)).astype(np.float32)
    c8 = DecodeChain(gpu, QWEN3_8B, batch=8, x_kind=BF16, seed=3, layers=2)
    assert c8.packed_hi
    gpu._check(gpu._lib.ingot_buffer_upload(gpu._h, c8.h_in.ptr, h0.ctypes.data, h0.nbytes))
    c8.step()
    gpu.complete()
    l8 = gpu.read_f32(c8.logits).reshape(8, -1)
    del c8
    c1 = DecodeChain(gpu, QWEN3_8B, batch=1, x_kind=BF16, seed=3, layers=2, fused_norm=False)
    gpu._check(gpu._lib.ingot_buffer_upload(gpu._h, c1.h_in.ptr, h0[3].ctypes.data, h0[3].nbytes))
    c1.step()
    gpu.complete()
    l1 = gpu.read_f32(c1.logits)
    scale = float(np.sqrt(np.mean(np.square(l1))))
    assert np.abs(l8[3] - l1).max() <= 2e-2 * scale


# ---- scratch and scopes around the wide-batch GEMM ------------------------------------------------

def test_wide_batch_projections_inside_an_independent_scope(gpu):
    # more than four tokens inside a scope: the GEMM's scratch is the handle's one workspace, so the scope takes the
    # GEMV in groups of four (the reference's project() runs for any count inside independent_projections, src/qwen.rs:822)
    cols, rows, tokens = 1024, 96, 8
    raws = [synth.random_matrix(Q4_K, cols, rows, seed=200 + i) for i in range(2)]
    ws = [gpu.bytes(r) for r in raws]
    x = standard_x(cols * tokens).reshape(tokens, cols)
    xb = gpu.floats(x)
    stride = synth.stride_of(Q4_K, cols)
    with gpu.independent():
        ys = [gpu.matmul(None, w, cols, rows, stride, Q4_K, 0, xb, tokens) for w in ws]
    got = [gpu.finish(None, y).reshape(tokens, rows) for y in ys]
    for g, raw in zip(got, raws):
        e = O.matvec_f64(raw, cols, rows, Q4_K, x)
        assert (np.abs(g - e) <= tol_ref(e)).all(), float(np.abs(g - e).max())


def test_recorded_command_survives_growth_of_the_scratch(gpu):
    # a recorded wide-batch projection has the scratch address in its kernel arguments; a later, larger call makes the
    # handle take a bigger scratch block, and the old block must stay valid for the replay
    cols, rows, tokens = 512, 128, 8
    raw = synth.random_matrix(Q4_K, cols, rows, seed=210)
    x = standard_x(cols * tokens).reshape(tokens, cols)
    w, xb, y = gpu.bytes(raw), gpu.floats(x), gpu.zeros(tokens * rows)
    stride = synth.stride_of(Q4_K, cols)
    gpu.matmul(None, w, cols, rows, stride, Q4_K, 0, xb, tokens, out=y)
    first = gpu.finish(None, y).copy()
    gpu.record()
    gpu.matmul(None, w, cols, rows, stride, Q4_K, 0, xb, tokens, out=y)
    graph = gpu.end_record()
    # a call whose scratch need (binary16 copy of 9000 x 4096 activations: 74 MB) exceeds the initial 16 MB block
    big_cols, big_rows, big_tokens = 4096, 128, 9000
    wb = gpu.bytes(synth.random_matrix(Q4_K, big_cols, big_rows, seed=211))
    xbig = gpu.zeros(big_tokens * big_cols)
    gpu.finish(None, gpu.gemm(None, wb, big_cols, big_rows, synth.stride_of(Q4_K, big_cols), Q4_K, 0, xbig, big_tokens))
    for _ in range(2):
        gpu._check(gpu._lib.ingot_buffer_zero(gpu._h, y.ptr, y.nbytes))
        graph.submit()
        assert np.array_equal(gpu.finish(None, y).view(np.uint32), first.view(np.uint32))


def test_wide_rows_keep_the_neighbours_of_an_outlier(gpu):
    """Two-digit fixed-point rows (the default when the norm rounds to bfloat16) give the 31 neighbours of an outlier
    300 times their size about 7 bits; INGOT_OPT_WIDE_ROWS builds four-digit rows instead.  The CPU restatement
    (tests/test_fixed_point_rows.py) puts the default at up to 1.7 times the reference's bound for this case."""
    from oracle.chain_check import expect_projection
    kind, cols, rows = Q4_K, 4096, 64
    raw = synth.random_matrix(kind, cols, rows, seed=cols + rows)
    a = synth.activations(1, cols, seed=2)
    a[0, 7] *= 300.0
    w, ab = gpu.bytes(raw), gpu.floats(a)
    stride = synth.stride_of(kind, cols)
    _, e, tol = expect_projection(raw, cols, rows, kind, a[0], None, True)
    worst = {}
    try:
        for wide in (0, 1):
            gpu.set_option(_abi.OPT_WIDE_ROWS, wide)
            y = gpu.output(rows)
            gpu._check(gpu._lib.ingot_matmul_normed(gpu._h, w.ptr, cols, rows, stride, kind, 0, ab.ptr, None, None, None, 1e-6, 0, 1, y.ptr))
            worst[wide] = float((np.abs(gpu.finish(None, y) - e) / tol).max())
    finally:
        gpu.set_option(_abi.OPT_WIDE_ROWS, 0)
    assert worst[1] <= 1.0, worst
    assert worst[0] <= 2.0 and worst[1] < worst[0], worst
