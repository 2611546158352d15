"""The streaming GEMV's plan, activation permutation and lane arithmetic, compiled
for the host (tests/host_emulation.cpp) and checked against the oracle.  This is the
same source the CUDA kernel is built from, so index or rounding mistakes show up here
before any GPU time is spent."""
import ctypes as C
import os
import subprocess

import numpy as np
import pytest

from conftest import ROOT, lcg_q4k_fixture, standard_x, tol_ref
from ingot_b200 import synth
from oracle import oracle as O

SO = os.path.join(ROOT, "tests", "_host_emulation.so")
SRC = os.path.join(ROOT, "tests", "host_emulation.cpp")
PLAN_FIELDS = ["kind", "cols", "rows", "stride", "units", "lpr_log2", "steps", "spc", "chunks", "chunk_bytes",
               "last_chunk_bytes", "tile_rows", "nmat", "ntok", "stages", "stage_bytes", "x_bytes", "smem_bytes",
               "ctas"]


@pytest.fixture(scope="module")
def em():
    deps = [SRC] + [os.path.join(ROOT, "ingot_b200", "csrc", f) for f in ("quant.cuh", "gemv_core.cuh")]
    if not os.path.exists(SO) or os.path.getmtime(SO) < max(map(os.path.getmtime, deps)):
        subprocess.run(["g++", "-O1", "-std=c++17", "-ffp-contract=off", "-fPIC", "-shared", "-o", SO, SRC],
                       check=True)
    lib = C.CDLL(SO)
    lib.emulate_gemv.restype = C.c_int
    assert lib.emulate_plan_words() == len(PLAN_FIELDS)
    return lib


def run(em, kind, raw, cols, rows, x, nmat=1, raw2=None, gelu=0, max_ctas=296, expert=0):
    x = np.ascontiguousarray(x, np.float32).reshape(-1, cols)
    y = np.zeros((x.shape[0], rows), np.float32)
    plan = np.zeros(len(PLAN_FIELDS), np.uint32)
    u8, f32, u32 = C.POINTER(C.c_uint8), C.POINTER(C.c_float), C.POINTER(C.c_uint32)
    r2 = raw if raw2 is None else raw2
    rc = em.emulate_gemv(kind, raw.ctypes.data_as(u8), r2.ctypes.data_as(u8), cols, rows, synth.stride_of(kind, cols),
                         expert, x.ctypes.data_as(f32), x.shape[0], nmat, gelu, max_ctas, y.ctypes.data_as(f32),
                         plan.ctypes.data_as(u32))
    return rc, y, dict(zip(PLAN_FIELDS, plan.tolist()))


SHAPES = {12: [(4096, 64), (2560, 37), (768, 33), (256, 7), (2048, 5), (1024, 1)],
          14: [(4096, 64), (2048, 5), (12288, 9)],
          2: [(4096, 64), (2560, 37), (768, 33), (256, 7), (10240, 3)],
          8: [(4096, 64), (2560, 37), (256, 7), (2048, 5)]}


@pytest.mark.parametrize("kind", [12, 14, 2, 8])
def test_emulated_kernel_matches_oracle(em, kind):
    for cols, rows in SHAPES[kind]:
        raw = synth.random_matrix(kind, cols, rows, seed=cols + rows)
        x = synth.activations(1, cols, seed=2)
        rc, y, plan = run(em, kind, raw, cols, rows, x)
        assert rc == 0, (kind, cols, rows)
        e = O.matvec_f64(raw, cols, rows, kind, x)
        assert (np.abs(y - e) <= tol_ref(e)).all(), (kind, cols, rows, np.abs(y - e).max())
        assert plan["smem_bytes"] <= 112 * 1024 and plan["stages"] >= 2
        assert plan["chunk_bytes"] % 16 == 0 and plan["last_chunk_bytes"] % 16 == 0
        assert (plan["chunks"] - 1) * plan["chunk_bytes"] + plan["last_chunk_bytes"] == plan["stride"]


def test_every_cta_split_gives_the_same_bits(em):
    # rows are independent: the CTA count must not change a single bit
    raw = synth.random_matrix(12, 2560, 41, seed=9)
    x = synth.activations(1, 2560, seed=1)
    base = run(em, 12, raw, 2560, 41, x, max_ctas=1)[1]
    for ctas in (2, 3, 7, 41, 296):
        assert np.array_equal(run(em, 12, raw, 2560, 41, x, max_ctas=ctas)[1].view(np.uint32), base.view(np.uint32))


@pytest.mark.parametrize("kind,cols", [(12, 2560), (14, 4096), (2, 2560), (8, 1024)])
def test_token_counts_agree_bitwise(em, kind, cols):
    # the reference's property: counts 2-4 bitwise equal to count 1 (kernels/iq3_mix.metal:81-84)
    rows = 37
    raw = synth.random_matrix(kind, cols, rows, seed=4)
    x = synth.activations(4, cols, seed=5)
    singles = np.stack([run(em, kind, raw, cols, rows, x[t:t + 1])[1][0] for t in range(4)])
    for n in (2, 3, 4):
        rc, y, _ = run(em, kind, raw, cols, rows, x[:n])
        if rc == 1 and n > 2:
            continue        # activations of n tokens do not fit beside the ring: the launcher regroups
        assert rc == 0
        assert np.array_equal(y.view(np.uint32), singles[:n].view(np.uint32))


def test_lcg_random_block_fixture(em):
    # src/expert_bench.rs:648-749: cols 2560, rows 37, 3 experts, expert 1, tol 1e-4 + 5e-5|e|
    data = lcg_q4k_fixture()
    x = standard_x(2560 * 4).reshape(4, 2560)
    rc, y, _ = run(em, 12, data, 2560, 37, x, expert=1)
    assert rc == 0
    e = O.matvec_f64(data, 2560, 37, 12, x, expert=1)
    assert (np.abs(y - e) <= tol_ref(e)).all()


@pytest.mark.parametrize("gelu", [0, 1])
def test_fused_gate_up_equals_separate(em, gelu):
    # src/metal/tests.rs "fused_gate_up_matches_separate": bitwise
    cols, rows = 2560, 19
    g, u = synth.random_matrix(2, cols, rows, seed=1), synth.random_matrix(2, cols, rows, seed=2)
    x = synth.activations(2, cols, seed=3)
    rc, fused, _ = run(em, 2, g, cols, rows, x, nmat=2, raw2=u, gelu=gelu)
    assert rc == 0
    yg, yu = run(em, 2, g, cols, rows, x)[1], run(em, 2, u, cols, rows, x)[1]
    sep = O.glu(yg, yu, gelu=bool(gelu))
    assert np.allclose(fused, sep, rtol=2e-6, atol=1e-7)
    e = O.glu(O.matvec_f64(g, cols, rows, 2, x).astype(np.float32), O.matvec_f64(u, cols, rows, 2, x).astype(np.float32),
              gelu=bool(gelu))
    assert np.abs(fused - e).max() <= 1e-4 + 1e-4 * np.abs(e).max()


def test_plan_falls_back_for_unaligned_rows(em):
    raw = synth.random_matrix(14, 256, 3, seed=0)          # stride 210: not a multiple of 16
    assert run(em, 14, raw, 256, 3, synth.activations(1, 256))[0] == 1


def test_scalar_decoder_in_kernel_header_matches_oracle(em):
    em.emulate_weight_at.restype = C.c_float
    for kind in (0, 1, 30, 2, 8, 12, 14):
        raw = synth.random_matrix(kind, 512, 1, seed=kind)
        want = O.dequant(raw, 512, 1, kind)[0]
        got = np.array([em.emulate_weight_at(raw.ctypes.data_as(C.POINTER(C.c_uint8)), kind, j) for j in range(512)],
                       np.float32)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
