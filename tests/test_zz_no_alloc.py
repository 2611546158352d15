"""The allocation-free entry point, `ingot_matvec_static`.

Some callers of this library cannot allocate device memory at all: a serving loop whose
host application has already given the rest of HBM to its KV cache, or a token step that
cannot take the device-wide synchronisation hidden in cudaMalloc/cudaFree.  For them the
library keeps the GEMV's scratch in a static device array.  This file checks that entry
point against the regular one (same kernels, so the same bits), twice in a row because
the scratch is shared between calls — once with an x the kernel can pack for itself and
once with an x that has to go through the static array — and that it refuses rows longer
than its scratch.
It is collected last so that a failure here cannot hide any other test.
"""
import ctypes as C

import numpy as np
import pytest

from ingot_b200 import Q4_K, Q6_K, _abi, synth
from oracle import oracle as O

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kind,cols,rows", [(Q4_K, 4096, 300), (Q6_K, 2048, 77)])
def test_static_scratch_matvec_matches_regular_entry_point_twice(gpu, kind, cols, rows):
    lib = _abi.load()
    stride = synth.stride_of(kind, cols)
    w = gpu.bytes(synth.random_matrix(kind, cols, rows, seed=21))
    for call in range(2):                                   # the second call reuses the same static scratch
        x = synth.activations(1, cols, seed=30 + call)
        xb = gpu.floats(x)
        want = gpu.finish(None, gpu.matmul(None, w, cols, rows, stride, kind, 0, xb, 1))
        y = gpu.zeros(rows)
        gpu.complete()
        st = lib.ingot_matvec_static(w.ptr, cols, rows, stride, kind, 0, xb.ptr, y.ptr, None, 1)
        assert st == _abi.OK, lib.ingot_matvec_static_error()
        got = gpu.read_f32(y)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("kind,cols,rows", [(Q4_K, 4096, 300), (Q6_K, 16384, 40)])
def test_static_scratch_holds_the_packed_row_of_an_unaligned_x_twice(gpu, kind, cols, rows):
    # an x that is only 4-byte aligned cannot be packed inside the kernel: a first launch packs it into the
    # static device array and the GEMV reads it from there.  Two calls in a row (the second over the first's
    # leftovers), the longest row the array holds among them, against the regular entry point on the same x.
    lib = _abi.load()
    stride = synth.stride_of(kind, cols)
    raw = synth.random_matrix(kind, cols, rows, seed=22)
    w = gpu.bytes(raw)
    for call in range(2):
        x = synth.activations(1, cols, seed=40 + call)
        shifted = gpu.floats(np.concatenate([np.zeros(1, np.float32), x[0]]))        # x starts 4 bytes into the buffer
        view = shifted.view_f32(1, cols)
        assert view.ptr % 16 == 4
        want = gpu.finish(None, gpu.matmul(None, w, cols, rows, stride, kind, 0, view, 1))
        y = gpu.zeros(rows)
        gpu.complete()
        st = lib.ingot_matvec_static(w.ptr, cols, rows, stride, kind, 0, view.ptr, y.ptr, None, 1)
        assert st == _abi.OK, lib.ingot_matvec_static_error()
        got = gpu.read_f32(y)
        # the regular entry point sends an unaligned x to another kernel, so the two agree to the GEMV bound
        # (|a - e| <= 1e-4 rms + 5e-5 |e| each against the f64 dot), not to the bit
        e = O.matvec_f64(raw, cols, rows, kind, x)[0]
        bound = 1e-4 * max(1.0, float(np.sqrt(np.mean(e * e)))) + 5e-5 * np.abs(e)
        assert (np.abs(got - e) <= bound).all(), float(np.abs(got - e).max())
        assert (np.abs(got - want) <= bound + 1e-3 * np.abs(e)).all()


def test_static_scratch_rejects_rows_beyond_its_size(gpu):
    lib = _abi.load()
    cols = 16384 + 256
    st = lib.ingot_matvec_static(C.c_void_p(16), cols, 1, synth.stride_of(Q4_K, cols), Q4_K, 0, C.c_void_p(16), C.c_void_p(16),
                                 None, 1)
    assert st == _abi.INVALID
    assert b"exceeds the static scratch" in lib.ingot_matvec_static_error()
    assert lib.ingot_matvec_static(C.c_void_p(16), 4096, 1, 100, Q4_K, 0, C.c_void_p(16), C.c_void_p(16), None, 1) == _abi.INVALID
