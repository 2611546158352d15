"""Row-sharded (tensor-parallel) decode step whose projections exchange their shards themselves: tagged
8-byte words stored into every rank's window, polled by the next projection (ingot_group_*).  Needs two GPUs with peer access;
both ranks live in this process (one handle per device, connected with ingot_group_connect_local).  A
rank's kernels wait only for kernels of the OTHER device, never for kernels of their own."""
import numpy as np
import pytest

from ingot_b200 import BF16

pytestmark = pytest.mark.gpu


def _device_count() -> int:
    try:
        import torch
        return torch.cuda.device_count()
    except Exception:
        return 0


@pytest.mark.skipif(_device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("recorded", [False, True], ids=["eager", "recorded"])
def test_sharded_step_with_peer_exchange_equals_the_unsharded_step(recorded):
    from ingot_b200 import Gpu
    from ingot_b200.chain import QWEN3_8B, DecodeChain
    from ingot_b200.gpu import Group
    layers, world = 2, 2
    h0 = np.random.default_rng(1).normal(0, 1, (1, QWEN3_8B.hidden)).astype(np.float32)
    g0 = Gpu(0)
    ref = DecodeChain(g0, QWEN3_8B, batch=1, x_kind=BF16, seed=3, layers=layers)
    g0._check(g0._lib.ingot_buffer_upload(g0._h, ref.h_in.ptr, h0.ctypes.data, h0.nbytes))
    ref.step()
    g0.complete()
    want = g0.read_f32(ref.logits).copy()
    del ref
    gpus = [g0, Gpu(1)]
    s = QWEN3_8B
    window = 4 * (s.q + 2 * s.hidden + s.ffn + s.vocab) + 8 * 256
    groups = [Group(g, r, world, window, DecodeChain.exchange_slots(layers)) for r, g in enumerate(gpus)]
    Group.connect_local(groups)
    chains = [DecodeChain(g, s, batch=1, x_kind=BF16, seed=3, layers=layers, rank=r, world=world, group=groups[r]) for r, g in enumerate(gpus)]
    for c, g in zip(chains, gpus):
        g._check(g._lib.ingot_buffer_upload(g._h, c.h_in.ptr, h0.ctypes.data, h0.nbytes))
        g.complete()
    if recorded:
        graphs = [c.record() for c in chains]
        steps = [gr.submit for gr in graphs]
    else:
        steps = [c.step for c in chains]
    for _ in range(3):                       # the same step three times: the tags move on with the step counter
        for c, g in zip(chains, gpus):
            g._check(g._lib.ingot_buffer_zero(g._h, c.logits.ptr, c.logits.nbytes))
            g.complete()
        for st in steps:                     # both ranks are issued before either is waited for
            st()
        for c, g in zip(chains, gpus):
            g.complete()
            got = g.read_f32(c.logits)
            assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    del chains
    for gr in groups:
        gr.close()
    gpus[1].close()
    g0.close()


def test_a_wait_nobody_answers_runs_out_and_reports_a_timeout():
    """Rank 0 of a group of two whose rank 1 never runs: the first projection that needs rank 1's rows gives up
    after its time limit (the later ones see the status and do not wait again), the handle reports the
    time-out and works on.  Both windows lie on one device here; only rank 0 issues kernels."""
    from ingot_b200 import DeviceTimeout, Gpu
    from ingot_b200.chain import QWEN3_8B, DecodeChain
    from ingot_b200.gpu import Group
    g = Gpu(0)
    s = QWEN3_8B
    window = 4 * (s.q + 2 * s.hidden + s.ffn + s.vocab) + 8 * 256
    groups = [Group(g, r, 2, window, DecodeChain.exchange_slots(1)) for r in range(2)]
    Group.connect_local(groups)
    chain = DecodeChain(g, s, batch=1, x_kind=BF16, seed=3, layers=1, rank=0, world=2, group=groups[0])
    chain.step()
    with pytest.raises(DeviceTimeout):
        g.complete()
    assert g.zeros(4).nbytes == 16           # the handle is usable after the time-out
    g.complete()
    del chain


@pytest.mark.skipif(_device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("grouped", [False, True], ids=["pair-by-pair", "grouped"])
@pytest.mark.parametrize("own_tokens", [1, 4, 16])
def test_token_all_to_all_equals_the_single_device_layers(own_tokens, grouped):
    """Two ranks, each with its own tokens and half of the experts: after two MoE layers with the token
    all-to-all every token's result is bit-identical to the layers run on one device that holds all experts,
    the received words are the ones the oracle's bookkeeping gives, and a second step repeats the first."""
    from ingot_b200 import Q4_K, Gpu
    from ingot_b200.gpu import EpExchange, Group
    from ingot_b200.moe import MoeChain, MoeShape
    from oracle import ep_exchange as X
    shape = MoeShape("test", 2, 512, 16, 4, 256, Q4_K)
    world, layers = 2, 2
    rng = np.random.default_rng(7)
    logits = rng.normal(0, 1, (world, own_tokens, shape.experts)).astype(np.float32)
    xs = (rng.normal(0, 1, (world, own_tokens, shape.hidden)) * 0.05).astype(np.float32)

    def load(c, r):
        g = c.gpu
        g._check(g._lib.ingot_buffer_upload(g._h, c.logits.ptr, logits[r].ctypes.data, logits[r].nbytes))
        g._check(g._lib.ingot_buffer_upload(g._h, c.x.ptr, xs[r].ctypes.data, xs[r].nbytes))
        g.complete()

    g0 = Gpu(0)
    want = []
    for r in range(world):                   # one device, all experts, the tokens of rank r, pair by pair
        ref = MoeChain(g0, shape, tokens=own_tokens, seed=3, layers=layers)
        ref.grouped = grouped
        load(ref, r)
        ref.step()
        g0.complete()
        want.append(g0.read_f32(ref.y).copy())
        del ref
    gpus = [g0, Gpu(1)]
    cap = own_tokens * shape.top
    window = EpExchange.window_bytes(world, cap, shape.hidden)
    groups = [Group(g, r, world, window, MoeChain.exchange_slots(layers)) for r, g in enumerate(gpus)]
    Group.connect_local(groups)
    chains = [MoeChain(g, shape, tokens=own_tokens, seed=3, layers=layers, rank=r, world=world, group=groups[r])
              for r, g in enumerate(gpus)]
    for r, c in enumerate(chains):
        c.grouped_places = grouped
        load(c, r)
    for _ in range(2):
        for c in chains:                     # both ranks are issued before either is waited for
            c.step()
        for r, (c, g) in enumerate(zip(chains, gpus)):
            g.complete()
            got = g.read_f32(c.y)
            assert np.array_equal(got.view(np.uint32), want[r].view(np.uint32))
    # the words of the last layer's receive areas against the oracle's plan (every layer routes the same logits)
    ids = [g.read_bytes(c.ids).view(np.uint32)[:cap] for c, g in zip(chains, gpus)]
    plans = [X.dispatch_plan(i, world, shape.experts // world, cap)[2] for i in ids]
    for r, (c, g) in enumerate(zip(chains, gpus)):
        region, ids_rx = X.receive_regions(plans, r)
        assert np.array_equal(g.read_bytes(c.ep.rx_meta).view(np.uint32)[:world * cap], region)
        assert np.array_equal(g.read_bytes(c.ids_rx).view(np.uint32), ids_rx)
    del chains


@pytest.mark.skipif(_device_count() < 2, reason="needs two GPUs")
@pytest.mark.xfail(strict=False, reason="written after this build's GPU time was spent: not yet run on two GPUs")
def test_one_group_takes_steps_of_different_token_counts():
    """Two MoE chains of different token counts on the SAME groups, one after the other: the exchange kernels' launches
    then differ in grid size from step to step, and the last-CTA counter of a launch must start from zero each time."""
    from ingot_b200 import Q4_K, Gpu
    from ingot_b200.gpu import EpExchange, Group
    from ingot_b200.moe import MoeChain, MoeShape
    shape = MoeShape("test", 2, 512, 16, 4, 256, Q4_K)
    world, layers = 2, 2
    counts = (16, 2, 5)
    rng = np.random.default_rng(8)
    logits = rng.normal(0, 1, (world, max(counts), shape.experts)).astype(np.float32)
    xs = (rng.normal(0, 1, (world, max(counts), shape.hidden)) * 0.05).astype(np.float32)

    def load(c, r, n):
        g = c.gpu
        g._check(g._lib.ingot_buffer_upload(g._h, c.logits.ptr, np.ascontiguousarray(logits[r][:n]).ctypes.data, 4 * n * shape.experts))
        g._check(g._lib.ingot_buffer_upload(g._h, c.x.ptr, np.ascontiguousarray(xs[r][:n]).ctypes.data, 4 * n * shape.hidden))
        g.complete()

    g0 = Gpu(0)
    want = []
    for r in range(world):                   # a token's result does not depend on the other tokens of its step
        ref = MoeChain(g0, shape, tokens=max(counts), seed=3, layers=layers)
        ref.grouped = False
        load(ref, r, max(counts))
        ref.step()
        g0.complete()
        want.append(g0.read_f32(ref.y).reshape(max(counts), shape.hidden).copy())
        del ref
    gpus = [g0, Gpu(1)]
    window = sum(EpExchange.window_bytes(world, n * shape.top, shape.hidden) for n in counts)
    groups = [Group(g, r, world, window, MoeChain.exchange_slots(layers)) for r, g in enumerate(gpus)]
    Group.connect_local(groups)
    for n in counts:
        chains = [MoeChain(g, shape, tokens=n, seed=3, layers=layers, rank=r, world=world, group=groups[r]) for r, g in enumerate(gpus)]
        for r, c in enumerate(chains):
            load(c, r, n)
        for c in chains:
            c.step()
        for r, (c, g) in enumerate(zip(chains, gpus)):
            g.complete()
            got = g.read_f32(c.y).reshape(n, shape.hidden)
            assert np.array_equal(got.view(np.uint32), want[r][:n].view(np.uint32)), n
        del chains

