"""The allocation-free entry point, `ingot_matvec_static`.

Some callers of this library cannot allocate device memory at all: a serving loop whose
host application has already given the rest of HBM to its KV cache, or a token step that
cannot take the device-wide synchronisation hidden in cudaMalloc/cudaFree.  For them the
library keeps the GEMV's scratch in a static device array.  This file checks that entry
point against the regular one (same kernels, so the same bits), twice in a row because
the scratch is shared between calls, and that it refuses rows longer than its scratch.
It is collected last so that a failure here cannot hide any other test.
"""
import ctypes as C

import numpy as np
import pytest

from ingot_b200 import Q4_K, Q6_K, _abi, synth

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


def test_static_scratch_rejects_rows_beyond_its_size(gpu):
    lib = _abi.load()
    cols = 16384 + 256
    st = lib.ingot_matvec_static(C.c_void_p(16), cols, 1, synth.stride_of(Q4_K, cols), Q4_K, 0, C.c_void_p(16), C.c_void_p(16),
                                 None, 1)
    assert st == _abi.INVALID
    assert b"exceeds the static scratch" in lib.ingot_matvec_static_error()
    assert lib.ingot_matvec_static(C.c_void_p(16), 4096, 1, 100, Q4_K, 0, C.c_void_p(16), C.c_void_p(16), None, 1) == _abi.INVALID
