"""GPU parity at the sizes of the benchmark configurations, through the entry points the
benchmark times: the fused-norm projections of the decode step (ingot_matmul_normed,
ingot_gate_up_normed, the grouped independent scope) on the Qwen3-8B and Gemma-3-4B shapes,
the two-layer chain against the oracle's own chain, the expert-routed GEMVs at 128 experts,
and the prefill GEMM on its K-split and wide-batch paths.  Every expectation is an f64 dot of
the dequantised weights (tests/projections.rs:37-46) on the inputs the operator read, with
the reference's bound |a - e| <= 1e-4 + 5e-5 |e| (absolute part scaled by the output RMS).
"""
import numpy as np
import pytest

from conftest import tol_contract, tol_ref_scaled
from ingot_b200 import BF16, F32, Q4_0, Q4_K, Q6_K, Tensor, Weight, synth
from oracle import chain_check as CK
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def normed(gpu, w, cols, rows, kind, a, b, bf16, s=None):
    y = gpu.output(rows)
    gpu._check(gpu._lib.ingot_matmul_normed(gpu._h, w.ptr, cols, rows, synth.stride_of(kind, cols), kind, 0, a.ptr,
                                            b.ptr if b else None, None, s.ptr if s else None, 1e-6, 1 if b else 0, int(bf16), y.ptr))
    return y


# (name, kind, cols, rows): the one-token projections of the two dense configurations that are
# launched alone (gate/up and the grouped q, k, v have tests of their own below)
SINGLE = [("qwen o / q", Q4_K, 4096, 4096), ("qwen down", Q6_K, 12288, 4096), ("qwen head", Q6_K, 4096, 151936),
          ("gemma o", Q4_0, 2048, 2560), ("gemma down", Q4_0, 10240, 2560), ("gemma head", Q4_0, 2560, 262144)]


@pytest.mark.parametrize("name,kind,cols,rows", SINGLE, ids=[s[0] for s in SINGLE])
@pytest.mark.parametrize("bf16", [1, 0], ids=["bf16", "f32"])
def test_normed_projection_at_config_size(gpu, name, kind, cols, rows, bf16):
    if rows > 100000 and not bf16:
        pytest.skip("the heads are checked with the benchmark's bfloat16 activations only")
    raw = synth.random_matrix(kind, cols, rows, seed=rows + cols)
    rng = np.random.default_rng(cols)
    a, b = rng.normal(0, 2, cols).astype(np.float32), rng.normal(0, 1, cols).astype(np.float32)
    w, ab, bb, sb = gpu.bytes(raw), gpu.floats(a), gpu.floats(b), gpu.output(cols)
    y = gpu.finish(None, normed(gpu, w, cols, rows, kind, ab, bb, bf16, sb)).astype(np.float64)
    s, e, tol = CK.expect_projection(raw, cols, rows, kind, a, b, bool(bf16))
    err = np.abs(y - e)
    assert (err <= tol).all(), (name, int(np.argmax(err / tol)), float((err / tol).max()))
    assert np.array_equal(gpu.read_f32(sb).view(np.uint32), s.view(np.uint32))
    w.release()


@pytest.mark.parametrize("kind,cols,rows,gelu", [(Q4_K, 4096, 12288, 0), (Q4_0, 2560, 10240, 1)], ids=["qwen", "gemma"])
@pytest.mark.parametrize("bf16", [1, 0], ids=["bf16", "f32"])
def test_gate_up_normed_at_config_size(gpu, kind, cols, rows, gelu, bf16):
    raw_g, raw_u = synth.random_matrix(kind, cols, rows, seed=11), synth.random_matrix(kind, cols, rows, seed=12)
    rng = np.random.default_rng(13)
    # inputs of model-like magnitude after the norm: gate and up outputs O(1..10), so the activation is not saturated
    a, b = rng.normal(0, 1, cols).astype(np.float32), rng.normal(0, 0.5, cols).astype(np.float32)
    wg, wu, ab, bb, sb, y = gpu.bytes(raw_g), gpu.bytes(raw_u), gpu.floats(a), gpu.floats(b), gpu.output(cols), gpu.output(rows)
    gpu._check(gpu._lib.ingot_gate_up_normed(gpu._h, wg.ptr, wu.ptr, cols, rows, synth.stride_of(kind, cols), kind, ab.ptr, bb.ptr,
                                             None, sb.ptr, 1e-6, 1, bf16, gelu, y.ptr))
    got = gpu.finish(None, y).astype(np.float64)
    s, e, tol = CK.expect_gate_up(raw_g, raw_u, cols, rows, kind, a, b, bool(bf16), bool(gelu))
    err = np.abs(got - e)
    assert (err <= tol).all(), (int(np.argmax(err / tol)), float((err / tol).max()))
    assert np.array_equal(gpu.read_f32(sb).view(np.uint32), s.view(np.uint32))


@pytest.mark.parametrize("shape", ["qwen", "gemma"])
def test_grouped_qkv_scope_at_config_size(gpu, shape):
    # q, k, v of one layer inside the independent scope: one grid of three parts, fused norm, bfloat16 rounding
    parts = ([(Q4_K, 4096, 4096), (Q4_K, 4096, 1024), (Q6_K, 4096, 1024)] if shape == "qwen"
             else [(Q4_0, 2560, 2048), (Q4_0, 2560, 1024), (Q4_0, 2560, 1024)])
    cols = parts[0][1]
    raws = [synth.random_matrix(k, c, r, seed=30 + i) for i, (k, c, r) in enumerate(parts)]
    ws = [gpu.bytes(r) for r in raws]
    rng = np.random.default_rng(31)
    a, b = rng.normal(0, 2, cols).astype(np.float32), rng.normal(0, 1, cols).astype(np.float32)
    ab, bb, sb = gpu.floats(a), gpu.floats(b), gpu.output(cols)
    with gpu.independent():
        ys = [normed(gpu, w, c, r, k, ab, bb, 1, sb if i == 0 else None) for i, (w, (k, c, r)) in enumerate(zip(ws, parts))]
    gpu.complete()
    for y, raw, (k, c, r) in zip(ys, raws, parts):
        s, e, tol = CK.expect_projection(raw, c, r, k, a, b, True)
        err = np.abs(gpu.read_f32(y).astype(np.float64) - e)
        assert (err <= tol).all(), (k, r, float((err / tol).max()))
    assert np.array_equal(gpu.read_f32(sb).view(np.uint32), s.view(np.uint32))


@pytest.mark.parametrize("x_kind", [BF16, F32], ids=["bf16", "f32"])
def test_two_layer_chain_operator_by_operator_and_logits(gpu, x_kind):
    # every operator of a two-layer Qwen3-8B-shaped step against the oracle on the inputs it read, the logits included
    from ingot_b200.chain import QWEN3_8B, DecodeChain
    chain = DecodeChain(gpu, QWEN3_8B, batch=1, x_kind=x_kind, seed=3, layers=2, keep_host=2)
    assert chain.fused_norm and chain.grouped_qkv
    h0 = np.random.default_rng(1).normal(0, 1, (1, QWEN3_8B.hidden)).astype(np.float32)
    gpu._check(gpu._lib.ingot_buffer_upload(gpu._h, chain.h_in.ptr, h0.ctypes.data, h0.nbytes))
    records = CK.check_fused_ops(gpu, chain, chain.fused_ops(), chain.host)
    assert len(records) == 2 * 6 + 1
    one_by_one = gpu.read_f32(chain.logits).copy()
    # the step as the benchmark issues it (grouped scope, one recorded command) gives the same logits bit for bit
    graph = chain.record()
    graph.submit()
    gpu.complete()
    assert np.array_equal(gpu.read_f32(chain.logits).view(np.uint32), one_by_one.view(np.uint32))
    # ... and so does the step as ONE persistent kernel (the chain), twice in a row
    fused = chain.record_chain()
    info = fused.info()
    assert info["projections"] == 13 and info["waits"] == 8 and info["stages"] >= 2, info
    for _ in range(2):
        gpu._check(gpu._lib.ingot_buffer_zero(gpu._h, chain.logits.ptr, chain.logits.nbytes))
        fused.submit()
        gpu.complete()
        assert np.array_equal(gpu.read_f32(chain.logits).view(np.uint32), one_by_one.view(np.uint32))
    if x_kind == F32:
        # without bfloat16 rounding points the oracle's own chain (f64 dots) reproduces the logits end to end
        e = CK.OracleChain(QWEN3_8B, layers=2, seed=3, bf16=False).step(h0[0]).astype(np.float64)
        assert (np.abs(one_by_one - e) <= 4 * tol_contract(e)).all(), float(np.abs(one_by_one - e).max())   # four chained GEMVs per layer


# ---- configuration 4: 128 experts ----------------------------------------------------------------

@pytest.mark.parametrize("tokens", [1, 8, 32])
def test_moe_layer_at_128_experts(gpu, tokens):
    from ingot_b200.moe import QWEN3_30B_A3B, MoeChain
    s = QWEN3_30B_A3B
    c = MoeChain(gpu, s, tokens=tokens, seed=5, layers=1, keep_host=True)
    rng = np.random.default_rng(40 + tokens)
    logits = rng.normal(0, 1, (tokens, s.experts)).astype(np.float32)
    x = (rng.normal(0, 1, (tokens, s.hidden)) * 0.05).astype(np.float32)
    gpu._check(gpu._lib.ingot_buffer_upload(gpu._h, c.logits.ptr, logits.ctypes.data, logits.nbytes))
    gpu._check(gpu._lib.ingot_buffer_upload(gpu._h, c.x.ptr, x.ctypes.data, x.nbytes))
    c.layer(0)
    y = gpu.finish(None, c.y).reshape(tokens, s.hidden)
    act = gpu.read_f32(c.act).reshape(tokens * s.top, s.ffn)
    out = gpu.read_f32(c.out).reshape(tokens * s.top, s.hidden)
    ids = gpu.read_u32(c.ids, tokens * s.top)
    wts = gpu.read_f32(c.w, tokens * s.top)
    ws = c.weights[0]
    # more than four tokens take the grouped path: act and out are then in packed (expert-major) order
    grouped = tokens > 4
    place = gpu.read_u32(c.inverse, tokens * s.top) if grouped else np.arange(tokens * s.top)
    if grouped:
        layout, tiles, packed, inverse, n_tiles = O.expert_layout(ids, s.experts, c.blocks)
        assert np.array_equal(place, inverse) and np.array_equal(gpu.read_u32(c.packed, tokens * s.top), packed)
        assert np.array_equal(gpu.read_u32(c.tiles, 4 * c.blocks).reshape(-1, 4), tiles)
        assert np.array_equal(gpu.read_u32(c.layout, 2 * s.experts).reshape(-1, 2), layout)
    for t in range(tokens):
        e_ids, e_w = O.route(logits[t], s.top)
        assert ids[t * s.top:(t + 1) * s.top].tolist() == e_ids.tolist()
        assert np.abs(wts[t * s.top:(t + 1) * s.top] - e_w).max() < 2e-6
        for j, k in enumerate(e_ids):
            p = int(place[t * s.top + j])
            eg = O.matvec_f64(ws["gate_host"], s.hidden, s.ffn, Q4_K, x[t], expert=int(k))[0]
            eu = O.matvec_f64(ws["up_host"], s.hidden, s.ffn, Q4_K, x[t], expert=int(k))[0]
            ea = O.glu(eg.astype(np.float32), eu.astype(np.float32)).astype(np.float64)
            assert (np.abs(act[p] - ea) <= tol_contract(ea)).all(), (t, j)
            ed = O.matvec_f64(ws["down_host"], s.ffn, s.hidden, Q4_K, act[p], expert=int(k))[0]      # the input the GPU's down projection read
            assert (np.abs(out[p] - ed) <= tol_ref_scaled(ed)).all(), (t, j)
        e_y = O.moe_sum(out[place[t * s.top:(t + 1) * s.top]], wts[t * s.top:(t + 1) * s.top], s.hidden, s.top)[0]
        assert np.abs(y[t] - e_y).max() <= 1e-6 * max(1.0, float(np.abs(e_y).max()))


# ---- configuration 5: prefill GEMM ---------------------------------------------------------------

def _sample_rows(rows):
    """First, last and tile-boundary rows (the GEMM's CTAs own 128 rows)."""
    picks = sorted({0, 1, 127, 128, 129, rows // 2 - 1, rows // 2, rows - 129, rows - 128, rows - 1})
    return [r for r in picks if 0 <= r < rows]


@pytest.mark.parametrize("kind,cols,rows,tokens", [(Q4_K, 4096, 12288, 512), (Q6_K, 12288, 4096, 512), (Q6_K, 12288, 4096, 2048),
                                                   (Q4_K, 4096, 12288, 2048)],
                         ids=["q4k-512", "q6k-512-ksplit", "q6k-2048", "q4k-2048"])
def test_gemm_at_config_size_on_sampled_rows(gpu, kind, cols, rows, tokens):
    raw = synth.random_matrix(kind, cols, rows, seed=50 + tokens)
    stride = synth.stride_of(kind, cols)
    x = synth.activations(tokens, cols, seed=51)
    xr = synth.from_bf16_bits(synth.to_bf16_bits(x))
    w, xb = gpu.bytes(raw), gpu.bf16(x)
    y = gpu.finish(None, gpu.gemm(None, w, cols, rows, stride, kind, 0, xb, tokens, BF16)).reshape(tokens, rows)
    picks = _sample_rows(rows)
    sub = np.concatenate([raw[r * stride:(r + 1) * stride] for r in picks])
    e = O.gemm_f16_f64(sub, cols, len(picks), kind, xr)                      # [tokens, picks]
    got = y[:, picks].astype(np.float64)
    rms = float(np.sqrt(np.mean(e * e)))
    assert (np.abs(got - e) <= 1e-4 * max(1.0, rms) + 5e-5 * np.abs(e)).all(), float(np.abs(got - e).max())
    # linearity over the whole output: y(x) at token 0 equals the one-token GEMV of the same row within the F16 staging error
    one = gpu.finish(None, gpu.matmul(None, w, cols, rows, stride, kind, 0, gpu.bf16(x[:1]), 1, BF16))
    scale = float(np.sqrt(np.mean(np.square(one))))
    assert np.abs(y[0] - one).max() <= 2e-3 * scale
    w.release()


def test_expert_projection_tile_tails(gpu):
    # the reference's tile fixture (src/metal/tests.rs:923-925, 2755-2776): tiles [expert, first, n, mode] =
    # [1,3,7,0] [0,10,16,1] [1,26,9,1] [0,35,1,1] [0,36,32,1] [1,68,19,1] over packed rows, pairs in reversed order;
    # packed rows outside the tiles stay as they were (zero), the others meet the f64 dot
    cols, rows, experts, top = 512, 65, 2, 2
    tiles = np.array([[1, 3, 7, 0], [0, 10, 16, 1], [1, 26, 9, 1], [0, 35, 1, 1], [0, 36, 32, 1], [1, 68, 19, 1], [0, 0, 0, 0]], np.uint32)
    total = 87
    pairs = np.arange(total, dtype=np.uint32)[::-1].copy()            # packed position q holds pair total - 1 - q
    raw = synth.random_matrix(Q4_K, cols, rows, experts, seed=60)
    w = gpu.bytes(raw)
    stride = synth.stride_of(Q4_K, cols)
    for gather in (1, 0):
        n_rows = (total + top - 1) // top if gather else total
        x = (synth.activations(n_rows, cols, seed=61 + gather) * np.float32(0.05)).astype(np.float32)
        y, xb, tb, pb = gpu.zeros(total * rows), gpu.floats(x), gpu.bytes(tiles), gpu.bytes(pairs)       # kept alive until the launch has run
        gpu._check(gpu._lib.ingot_expert_project(gpu._h, w.ptr, cols, rows, stride, Q4_K, experts, xb.ptr, tb.ptr, pb.ptr, len(tiles), top,
                                                 total, gather, y.ptr))
        got = gpu.finish(None, y).reshape(total, rows)
        covered = np.zeros(total, bool)
        for e, first, n, _ in tiles:
            for q in range(first, first + n):
                covered[q] = True
                src = int(pairs[q]) // top if gather else q
                want = O.matvec_f64(raw, cols, rows, Q4_K, x[src], expert=int(e))[0]
                assert (np.abs(got[q] - want) <= tol_ref_scaled(want)).all(), (gather, q)
        assert not got[~covered].any()
    # an expert id beyond the matrix is an error code, not a fault
    bad = np.array([[2, 0, 1, 0]], np.uint32)
    xb, tb, pb, yb = gpu.zeros(cols), gpu.bytes(bad), gpu.bytes(pairs), gpu.zeros(total * rows)
    gpu._check(gpu._lib.ingot_expert_project(gpu._h, w.ptr, cols, rows, stride, Q4_K, experts, xb.ptr, tb.ptr, pb.ptr, 1, top, total, 0, yb.ptr))
    from ingot_b200 import InvalidData
    with pytest.raises(InvalidData):
        gpu.complete()


def test_moe_layer_at_prefill_width_takes_the_per_expert_gemms(gpu):
    """More than 256 tokens: rows gathered into packed order, every expert's run through the tensor-core GEMM
    (Generic::moe_packed, src/generic.rs:578-660).  The GEMM stages weights and activations in binary16, as the
    reference's does, so the layer is compared with the pair-by-pair GEMV result within that staging's noise
    (three chained projections: 1e-3 of full precision each, src/expert_bench.rs:734-749), and the bookkeeping —
    every packed row belongs to the expert and the token the tables say — exactly."""
    from ingot_b200.moe import MoeChain, MoeShape
    from ingot_b200 import Q4_K
    shape = MoeShape("test", 1, 512, 16, 4, 256, Q4_K)
    tokens = 300
    rng = np.random.default_rng(77)
    logits = rng.normal(0, 1, (tokens, shape.experts)).astype(np.float32)
    x = (rng.normal(0, 1, (tokens, shape.hidden)) * 0.05).astype(np.float32)
    results = []
    for grouped in (False, True):
        c = MoeChain(gpu, shape, tokens=tokens, seed=9, layers=1)
        c.grouped = grouped
        gpu._check(gpu._lib.ingot_buffer_upload(gpu._h, c.logits.ptr, logits.ctypes.data, logits.nbytes))
        gpu._check(gpu._lib.ingot_buffer_upload(gpu._h, c.x.ptr, x.ctypes.data, x.nbytes))
        c.layer(0)
        results.append(gpu.finish(None, c.y).reshape(tokens, shape.hidden).copy())
        if grouped:
            pairs = tokens * shape.top
            ids = gpu.read_u32(c.ids, pairs)
            packed, layout = gpu.read_u32(c.packed, pairs), gpu.read_u32(c.layout, 2 * shape.experts).reshape(-1, 2)
            xp = gpu.read_f32(c.x_packed).reshape(pairs, shape.hidden)
            assert np.array_equal(xp.view(np.uint32), x[packed // shape.top].view(np.uint32))
            for e, (n, first) in enumerate(layout):
                assert (ids[packed[first:first + n]] == e).all()
        del c
    plain, gemm = results
    scale = float(np.abs(plain).max())
    assert np.abs(gemm - plain).max() <= 1e-2 * scale, float(np.abs(gemm - plain).max() / scale)
