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
