"""The operators around the projections in a generic decode step — embedding rows, rotary embedding
with the cache write, decode attention, greedy choice — against their oracle restatements
(kernels/qwen.metal:139, kernels/generic.metal:405-474, kernels/qwen.metal:384-410), and a whole
two-layer token step assembled from them and the projections (Generic::hidden,
src/generic.rs:664-749) against the same graph run on the oracle."""
import numpy as np
import pytest

from ingot_b200 import BF16, F16, F32, Q4_0, Q4_K, Q6_K, Q8_0, InvalidData, Tensor, Weight, synth
from oracle import oracle as O

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kind", [F32, F16, BF16, Q4_0, Q8_0, Q4_K, Q6_K])
def test_embedding_rows_are_bit_exact(gpu, kind):
    width, vocab = 512, 97
    raw = synth.random_matrix(kind, width, vocab, seed=kind + 1)
    t = Tensor.of([width, vocab], kind)
    w = Weight(gpu.bytes(raw), t)
    ids = np.array([0, 96, 5, 5, 42], np.uint32)
    got = gpu.finish(None, gpu.embedding_batch(None, w, gpu.bytes(ids), ids.size)).reshape(ids.size, width)
    want = O.embedding(raw, ids, width, vocab, kind)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    gpu.embedding_batch(None, w, gpu.bytes(np.array([97], np.uint32)), 1)        # outside the vocabulary: an error, not a fault
    with pytest.raises(InvalidData):
        gpu.complete()


@pytest.mark.parametrize("neox,qk_norm,factors,value_norm", [(False, False, False, False), (True, True, False, False), (True, True, True, True)])
@pytest.mark.parametrize("D,H,KV,rot", [(128, 8, 2, 128), (256, 4, 2, 128), (64, 6, 3, 32)])
def test_qk_rope_cache(gpu, D, H, KV, rot, neox, qk_norm, factors, value_norm):
    tokens, position, rows = 3, 17, 32
    rng = np.random.default_rng(D + H)
    q, k, v = (rng.normal(0, 1, (tokens, n, D)).astype(np.float32) for n in (H, KV, KV))
    qn, kn = (rng.normal(1, 0.1, D).astype(np.float32) for _ in range(2))
    fac = rng.uniform(0.5, 2.0, rot // 2).astype(np.float32)
    kc0, vc0 = (rng.normal(0, 1, (rows, KV, D)).astype(np.float32) for _ in range(2))
    kcb, vcb, qob = gpu.floats(kc0), gpu.floats(vc0), gpu.output(tokens * H * D)
    gpu.qk_rope_cache(None, gpu.floats(q), gpu.floats(k), gpu.floats(v), qob, kcb, vcb, head_dim=D, heads=H, kv_heads=KV, rotated=rot,
                      position=position, base=1e6, tokens=tokens, neox=neox, factors=gpu.floats(fac) if factors else None,
                      q_norm=gpu.floats(qn) if qk_norm else None, k_norm=gpu.floats(kn) if qk_norm else None, eps=1e-6,
                      value_norm=value_norm, q_scale=0.25)
    got_q = gpu.finish(None, qob).reshape(tokens, H, D)
    kc, vc = kc0.copy(), vc0.copy()
    want_q = O.qk_rope_cache(q, k, v, kc, vc, head_dim=D, heads=H, kv_heads=KV, rotated=rot, position=position, base=1e6, tokens=tokens,
                             neox=neox, factors=fac if factors else None, q_norm=qn if qk_norm else None, k_norm=kn if qk_norm else None,
                             eps=1e-6, value_norm=value_norm, q_scale=0.25)
    got_k, got_v = gpu.read_f32(kcb).reshape(rows, KV, D), gpu.read_f32(vcb).reshape(rows, KV, D)
    # float32 angle and trigonometry against the oracle's float64: position * base^(-2f/rot) up to 19, ulp 2e-6
    assert np.abs(got_q - want_q).max() <= 2e-5 and np.abs(got_k - kc).max() <= 4e-5 and np.abs(got_v - vc).max() <= 2e-6
    untouched = np.r_[0:position, position + tokens:rows]
    assert np.array_equal(got_k[untouched], kc0[untouched]) and np.array_equal(got_v[untouched], vc0[untouched])


@pytest.mark.parametrize("D,H,KV", [(128, 32, 8), (256, 8, 4), (64, 4, 4), (96, 6, 2), (512, 2, 1)])
@pytest.mark.parametrize("position,tokens,window", [(0, 1, 0), (5, 4, 0), (300, 2, 0), (300, 3, 128)])
def test_attention_decode(gpu, D, H, KV, position, tokens, window):
    rows = position + tokens
    rng = np.random.default_rng(D + position)
    q = rng.normal(0, 1, (tokens, H, D)).astype(np.float32)
    kc, vc = (rng.normal(0, 1, (rows, KV, D)).astype(np.float32) for _ in range(2))
    out = gpu.attention_decode(None, gpu.floats(q), gpu.floats(kc), gpu.floats(vc), D, H, KV, position, tokens, window)
    got = gpu.finish(None, out).reshape(tokens, H, D)
    want = O.attention_decode(q, kc, vc, D, H, KV, position, tokens, window)
    assert np.abs(got - want).max() <= 2e-5, float(np.abs(got - want).max())


@pytest.mark.parametrize("D,H,KV,position,rows,window", [(64, 8, 2, 0, 40, 0), (128, 4, 4, 57, 70, 0), (128, 8, 2, 100, 33, 48),
                                                        (256, 2, 1, 3, 9, 0), (96, 4, 2, 0, 130, 64)])
def test_attention_prefill(gpu, D, H, KV, position, rows, window):
    # what the reference runs for more than four tokens (flash_prefill_<D>): the tails of its 8-row and 64-key tiles
    # (rows and lengths that are no multiples) are ordinary cases here
    length = position + rows
    rng = np.random.default_rng(D + rows)
    q = rng.normal(0, 1, (rows, H, D)).astype(np.float32)
    kc, vc = (rng.normal(0, 1, (length, KV, D)).astype(np.float32) for _ in range(2))
    out = gpu.attention_prefill(None, gpu.floats(q), gpu.floats(kc), gpu.floats(vc), D, H, KV, position, rows, window)
    got = gpu.finish(None, out).reshape(rows, H, D)
    want = O.attention_decode(q, kc, vc, D, H, KV, position, rows, window)
    assert np.abs(got - want).max() <= 2e-5, float(np.abs(got - want).max())
    with pytest.raises(InvalidData):            # rows beyond the stated length
        gpu._check(gpu._lib.ingot_attention_prefill(gpu._h, out.ptr, out.ptr, out.ptr, out.ptr, D, H, KV, length - 1, position, rows, window))


def test_architecture_glue(gpu):
    # kernels/generic_arch.metal:2-17: scale, logit soft-cap, SwiGLU over fused gate|up rows, column copy
    rng = np.random.default_rng(5)
    x = rng.normal(0, 4, 3 * 1000).astype(np.float32)
    xb = gpu.floats(x)
    got = gpu.finish(None, gpu.scale_rows(None, xb, x.size, 0.0625 * 3))
    assert np.array_equal(got.view(np.uint32), O.scale_rows(x, 0.0625 * 3).view(np.uint32))
    got, want = gpu.finish(None, gpu.softcap_rows(None, xb, x.size, 30.0)), O.softcap_rows(x, 30.0)
    assert np.abs(got - want).max() <= 4e-6 * 30.0
    got, want = gpu.finish(None, gpu.swiglu_fused(None, xb, 3, 500)).reshape(3, 500), O.swiglu_fused(x, 3, 500)
    assert (np.abs(got - want) <= 2e-6 * np.abs(want) + 1e-7).all(), float(np.abs(got - want).max())
    got = gpu.finish(None, gpu.copy_columns(None, xb, 3, 77, 123, 1000)).reshape(3, 77)
    assert np.array_equal(got.view(np.uint32), O.copy_columns(x, 3, 77, 123, 1000).view(np.uint32))
    assert gpu.finish(None, gpu.copy_columns(None, xb, 3, 1000, 0, 1000)).size == 3000            # whole rows
    with pytest.raises(InvalidData):
        gpu.copy_columns(None, xb, 3, 77, 950, 1000)                                               # columns past the row
    with pytest.raises(InvalidData):
        gpu.softcap_rows(None, xb, x.size, 0.0)


def test_attention_decode_without_a_kernel_is_unsupported(gpu):
    z = gpu.zeros(4 * 80)
    assert gpu.attention_decode(None, z, z, z, 80, 4, 4, 0, 1) is None


def test_greedy_select(gpu):
    vocab, rows = 151936, 3
    rng = np.random.default_rng(3)
    logits = rng.normal(0, 1, (rows, vocab)).astype(np.float32)
    logits[0, 7] = logits[0, 150000] = 9.0                 # a tie: the smaller token wins
    logits[1, 1000] = 0.0; logits[1] = np.minimum(logits[1], 0.0); logits[1, 5000] = -0.0      # signed zeros tie by id
    lb = gpu.floats(logits)
    got = gpu.finish_greedy(None, lb, rows, vocab)
    want = O.greedy(logits, vocab)
    assert got == want[:, 0].tolist() and got[0] == 7
    mapping = rng.permutation(vocab).astype(np.uint32)
    got = gpu.finish_greedy(None, lb, rows, vocab, gpu.bytes(mapping))
    assert got == O.greedy(logits, vocab, mapping)[:, 0].tolist()
    small = rng.normal(0, 1, (2, 100)).astype(np.float32)
    assert gpu.finish_greedy(None, gpu.floats(small), 2, 100) == small.argmax(axis=1).tolist()
    small[1, 3] = np.nan
    with pytest.raises(InvalidData):
        gpu.finish_greedy(None, gpu.floats(small), 2, 100)


def test_whole_token_step_matches_the_oracle_graph(gpu):
    # Generic::hidden at decode for a two-layer Qwen3-shaped model (hidden 512, 8 heads of 64, 2 KV heads, FFN 1024,
    # QK norm, NeoX rotary embedding): embedding -> [add_rms -> q, k, v -> rope + cache -> attention -> o -> add_rms ->
    # gate/up + SiLU -> down] x 2 -> add_rms -> head -> greedy, two tokens one after the other, against the same graph of
    # oracle operators on the same weights
    hidden, heads, kvh, D, ffn, vocab, layers, rows = 512, 8, 2, 64, 1024, 1000, 2, 8
    rng = np.random.default_rng(11)
    def mk(kind, cols, rws, seed):
        raw = synth.random_matrix(kind, cols, rws, seed=seed)
        return raw, Weight(gpu.bytes(raw), Tensor.of([cols, rws], kind))
    emb = mk(Q4_K, hidden, vocab, 1)
    head = mk(Q6_K, hidden, vocab, 2)
    L = []
    for i in range(layers):
        L.append({"q": mk(Q4_K, hidden, heads * D, 10 * i + 3), "k": mk(Q4_K, hidden, kvh * D, 10 * i + 4), "v": mk(Q6_K, hidden, kvh * D, 10 * i + 5),
                  "o": mk(Q4_K, heads * D, hidden, 10 * i + 6), "gate": mk(Q4_K, hidden, ffn, 10 * i + 7), "up": mk(Q4_K, hidden, ffn, 10 * i + 8),
                  "down": mk(Q6_K, ffn, hidden, 10 * i + 9),
                  "attn_norm": rng.normal(1, 0.1, hidden).astype(np.float32), "ffn_norm": rng.normal(1, 0.1, hidden).astype(np.float32),
                  "qn": rng.normal(1, 0.1, D).astype(np.float32), "kn": rng.normal(1, 0.1, D).astype(np.float32)})
    out_norm = rng.normal(1, 0.1, hidden).astype(np.float32)
    kc = [np.zeros((rows, kvh, D), np.float32) for _ in range(layers)]
    vc = [np.zeros((rows, kvh, D), np.float32) for _ in range(layers)]
    kcb, vcb = [gpu.floats(c) for c in kc], [gpu.floats(c) for c in vc]

    def mv(pair, x):
        raw, w = pair
        return O.matvec_f64(raw, w.t.dims[0], w.t.dims[1], w.t.kind, np.asarray(x, np.float32).reshape(1, -1))[0].astype(np.float32)

    def oracle_step(token, position):
        x = O.embedding(emb[0], [token], hidden, vocab, Q4_K)[0] * np.float32(0.05)
        delta = None
        for i, l in enumerate(L):
            x, n = O.add_rms(x, delta if delta is not None else x, l["attn_norm"], 1e-6, add=delta is not None)
            q, k, v = mv(l["q"], n), mv(l["k"], n), mv(l["v"], n)
            qo = O.qk_rope_cache(q, k, v, kc[i], vc[i], head_dim=D, heads=heads, kv_heads=kvh, rotated=D, position=position, base=1e6,
                                 tokens=1, neox=True, q_norm=l["qn"], k_norm=l["kn"], eps=1e-6)
            a = O.attention_decode(qo, kc[i], vc[i], D, heads, kvh, position, 1).reshape(-1)
            x, n = O.add_rms(x, mv(l["o"], a), l["ffn_norm"], 1e-6)
            delta = mv(l["down"], O.glu(mv(l["gate"], n), mv(l["up"], n)))
        x, n = O.add_rms(x, delta, out_norm, 1e-6)
        return mv(head, n)

    def gpu_step(token, position):
        ids = gpu.bytes(np.array([token], np.uint32))
        x = gpu.embedding_batch(None, emb[1], ids, 1)
        xs = gpu.floats(gpu.finish(None, x) * np.float32(0.05))         # the embedding scale (scale_rows) on the host: not an operator of this path
        delta = None
        for i, l in enumerate(L):
            if delta is None:
                x2, n = xs, gpu.add_rms(None, xs, None, gpu.floats(l["attn_norm"]), hidden, 1, 1e-6, add=False)[1]
            else:
                x2, n = gpu.add_rms(None, xs, delta, gpu.floats(l["attn_norm"]), hidden, 1, 1e-6)
            with gpu.independent():
                q, k, v = (gpu.generic_project(None, l[r][1], n, 1) for r in ("q", "k", "v"))
            qo = gpu.output(heads * D)
            gpu.qk_rope_cache(None, q, k, v, qo, kcb[i], vcb[i], head_dim=D, heads=heads, kv_heads=kvh, rotated=D, position=position,
                              base=1e6, tokens=1, neox=True, q_norm=gpu.floats(l["qn"]), k_norm=gpu.floats(l["kn"]), eps=1e-6)
            a = gpu.attention_decode(None, qo, kcb[i], vcb[i], D, heads, kvh, position, 1)
            o = gpu.generic_project(None, l["o"][1], a, 1)
            xs, n = gpu.add_rms(None, x2, o, gpu.floats(l["ffn_norm"]), hidden, 1, 1e-6)
            act = gpu.generic_gate_up(None, [l["gate"][1], l["up"][1]], n, 1, False)
            delta = gpu.generic_project(None, l["down"][1], act, 1)
        _, n = gpu.add_rms(None, xs, delta, gpu.floats(out_norm), hidden, 1, 1e-6)
        logits = gpu.generic_project(None, head[1], n, 1)
        return gpu.finish(None, logits), gpu.finish_greedy(None, logits, 1, vocab)[0]

    for position, token in enumerate([17, 503]):
        e = oracle_step(token, position).astype(np.float64)
        got, choice = gpu_step(token, position)
        rms = float(np.sqrt(np.mean(e * e)))
        # nine chained projections and two attentions: the GEMV bound (1e-4 rms + 5e-5 |e|) per link, four of them deep
        assert (np.abs(got - e) <= 4 * (1e-4 * max(1.0, rms) + 5e-5 * np.abs(e)) + 1e-3 * np.abs(e)).all(), float(np.abs(got - e).max())
        assert choice == int(np.argmax(got))
