"""The size-keyed pool of output buffers behind Gpu::output / configure_workspace (src/metal.rs:1278-1342), with the
cases of the reference's workspace tests (src/metal/tests.rs:1244-1346), and Gpu::ffn on device buffers."""
import numpy as np
import pytest

from ingot_b200 import Q4_K, InvalidData, Matrix, synth
from oracle import oracle as O

pytestmark = pytest.mark.gpu
PAGE = 16 * 1024


@pytest.fixture()
def gpu():
    from ingot_b200 import Gpu
    g = Gpu(0)
    yield g
    g.close()


def test_pressure_keeps_unneeded_idle_buffers_reusable(gpu):
    gpu.configure_workspace(5 * PAGE)
    small, large, live = gpu.output(4), gpu.output(3 * PAGE // 4), gpu.output(5)
    small.release()
    large.release()
    before = gpu.workspace_statistics()[0]
    medium = gpu.output(2 * PAGE // 4)          # needs the large idle buffer's room, not the small one's
    small_again = gpu.output(4)
    assert gpu.workspace_statistics()[0] == before + 1
    assert gpu.workspace_statistics()[2] <= 5 * PAGE
    for b in (live, medium, small_again):
        b.release()


def test_bounded_and_evicts_unused_sizes(gpu):
    gpu.configure_workspace(2 * PAGE)
    first, second = gpu.output(4), gpu.output(5)
    with pytest.raises(InvalidData, match="workspace live allocation exceeds budget"):
        gpu.output(6)                          # the live set must fit the budget
    first.release()
    third = gpu.output(6)
    assert gpu.workspace_statistics()[2] == 2 * PAGE
    second.release()
    third.release()
    gpu.output(7).release()
    before = gpu.workspace_statistics()[0]
    gpu.output(7).release()
    assert gpu.workspace_statistics()[0] == before
    zero = gpu.zeros(4)                        # persistent state bypasses the pool
    assert np.array_equal(gpu.read_f32(zero), np.zeros(4, dtype=np.float32))
    assert gpu.workspace_statistics()[0] == before


def test_released_buffers_are_reused_in_stream_order(gpu):
    """A released buffer is handed out again at once: work enqueued on it earlier runs first on the handle's stream."""
    gpu.configure_workspace(8 * PAGE)
    first = gpu.output(4)
    address = first.ptr
    first.release()
    again = gpu.output(4)
    assert again.ptr == address and gpu.workspace_statistics()[1] == 1
    again.release()
    before = gpu.workspace_statistics()[0]
    for _ in range(100):
        gpu.output(4).release()
    assert gpu.workspace_statistics()[0] == before


def test_a_buffer_goes_back_to_the_pool_once(gpu):
    gpu.configure_workspace(4 * PAGE)
    b = gpu.output(16)
    ptr = b.ptr
    b.release()
    assert gpu._lib.ingot_output_release(gpu._h, ptr) != 0          # a second release is refused, not queued twice
    c, d = gpu.output(16), gpu.output(16)
    assert c.ptr == ptr and d.ptr != ptr
    c.release()
    d.release()


def test_without_a_budget_outputs_are_plain_allocations(gpu):
    x = gpu.output(1000)
    assert gpu.workspace_statistics() == (0, 0, 0, 0)
    x.release()
    with pytest.raises(InvalidData):
        gpu.output(0)


def test_ffn_of_stacked_experts_matches_the_oracle(gpu):
    width, inner, count = 512, 256, 3
    mats = []
    for i, (cols, rows) in enumerate(((width, inner), (width, inner), (inner, width))):
        raw = synth.random_matrix(Q4_K, cols, rows, count, seed=40 + i)
        mats.append(Matrix(raw, cols, rows, count, Q4_K, synth.stride_of(Q4_K, cols)))
    x = (np.random.default_rng(1).normal(0, 1, width) * 0.05).astype(np.float32)
    got = gpu.read_f32(gpu.ffn(mats, gpu.floats(x))).reshape(count, width)
    for e in range(count):
        act = O.glu(O.matvec_f64(mats[0].data, width, inner, Q4_K, x, expert=e)[0].astype(np.float32),
                    O.matvec_f64(mats[1].data, width, inner, Q4_K, x, expert=e)[0].astype(np.float32))
        want = O.matvec_f64(mats[2].data, inner, width, Q4_K, act, expert=e)[0]
        assert np.abs(got[e] - want).max() <= 1e-4 * max(1.0, float(np.sqrt(np.mean(want * want)))) + 5e-5 * np.abs(want).max()
