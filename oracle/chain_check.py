"""Checker for the dense decode chain: the oracle's own token step and a per-operator
comparison of the CUDA chain against it.  Test infrastructure only: used by tests/, by
__graft_entry__.smoke() and by bench.py (the parity check outside the timed region and
the CPU baseline); the product package never imports it.

The chain's dataflow is the projection skeleton of the reference's Generic::hidden
(src/generic.rs:664-763) with add_rms (kernels/generic.metal:390-404) between the
projections; see ingot_b200/chain.py for the stand-ins it uses.  Every projection is
y = W . round(rms_norm(a + b)), checked against an f64 dot of the dequantised weights
(tests/projections.rs:37-46) on the SAME inputs a, b that the CUDA operator read.
"""
from __future__ import annotations

import numpy as np

from . import oracle as O

EPS = 1e-6
ROLE_ORDER = ("q", "k", "v", "o", "gate", "up", "down")


def bf16_round(x: np.ndarray) -> np.ndarray:
    return O.from_bf16_bits(O.to_bf16_bits(np.ascontiguousarray(x, np.float32)))


def normalised_input(a: np.ndarray, b: np.ndarray | None, bf16: bool):
    """(sum, x, ambiguous): the float32 residual sum a + b, the activation row the projection reads
    (rms_norm in float64, rounded to float32 and then to bfloat16 when `bf16`), and the indices whose
    bfloat16 rounding depends on the last few float32 bits of the normalised value: a float32
    evaluation of the norm, in any summation order, may round those the other way."""
    s = a.astype(np.float32) + (b.astype(np.float32) if b is not None else np.float32(0))
    s64 = s.astype(np.float64)
    inv = 1.0 / np.sqrt(np.mean(s64 * s64) + EPS)
    x32 = (s64 * inv).astype(np.float32)
    if not bf16:
        return s, x32, np.zeros(0, np.int64)
    frac = (x32.view(np.uint32) & 0xFFFF).astype(np.int64)
    ambiguous = np.nonzero(np.abs(frac - 0x8000) <= 16)[0]      # within 16 float32 ulps of a rounding midpoint
    return s, bf16_round(x32), ambiguous


def rounding_slack(raw, cols, rows, kind, x: np.ndarray, ambiguous: np.ndarray) -> np.ndarray:
    """Per output row, the most the result can move when the ambiguous activations round the other
    way: sum over them of |W[r][i]| * (one bfloat16 step of x[i])."""
    if ambiguous.size == 0:
        return np.zeros(rows)
    steps = np.zeros((ambiguous.size, cols), np.float32)
    for j, i in enumerate(ambiguous):
        v = np.float32(x[i])
        exp = (v.view(np.uint32) >> 23) & 0xFF
        steps[j, i] = np.float32(2.0 ** (int(exp) - 127 - 7)) if exp else np.float32(2.0 ** -133)
    return np.abs(O.matvec_f64(raw, cols, rows, kind, steps)).sum(axis=0)


def tol_ref_scaled(e: np.ndarray) -> np.ndarray:
    """The reference's GEMV bound |a - e| <= 1e-4 + 5e-5 |e| (tests/projections.rs:42-46), its
    absolute part scaled by the output RMS when that exceeds 1 (synthetic blocks give outputs of
    magnitude ~300, where float32 summation alone exceeds 1e-4 absolute)."""
    rms = float(np.sqrt(np.mean(np.square(e)))) if e.size else 0.0
    return 1e-4 * max(1.0, rms) + 5e-5 * np.abs(e)


def expect_projection(raw, cols, rows, kind, a, b, bf16: bool):
    """(sum, expected f64 [rows], tolerance [rows]) of y = W . round(rms_norm(a + b))."""
    s, x, amb = normalised_input(a, b, bf16)
    e = O.matvec_f64(raw, cols, rows, kind, x.reshape(1, cols))[0]
    return s, e, tol_ref_scaled(e) + rounding_slack(raw, cols, rows, kind, x, amb)


def expect_gate_up(raw_g, raw_u, cols, rows, kind, a, b, bf16: bool, gelu: bool):
    """The same for act = glu(gate . x, up . x): the two projections' bounds carried through the
    activation (|d act| <= |glu'(g)| |u| dg + |act / u| du) plus float32 rounding of the activation."""
    s, x, amb = normalised_input(a, b, bf16)
    eg = O.matvec_f64(raw_g, cols, rows, kind, x.reshape(1, cols))[0]
    eu = O.matvec_f64(raw_u, cols, rows, kind, x.reshape(1, cols))[0]
    tg = tol_ref_scaled(eg) + rounding_slack(raw_g, cols, rows, kind, x, amb)
    tu = tol_ref_scaled(eu) + rounding_slack(raw_u, cols, rows, kind, x, amb)
    act = O.glu(eg.astype(np.float32), eu.astype(np.float32), gelu).astype(np.float64)
    gated = np.where(eu != 0, np.abs(act / np.where(eu != 0, eu, 1.0)), np.abs(eg))      # |silu(g)| or |gelu(g)|
    tol = 1.13 * np.abs(eu) * tg + (gated + 1.13 * tg) * tu + 4e-6 * np.abs(act) + 1e-30
    return s, act, tol


def check_fused_ops(gpu, chain, ops, host_weights) -> list[dict]:
    """Issues `ops` (ingot_b200.chain.FusedOp) one at a time, in order, and compares each result with
    the oracle's expectation for the inputs the operator actually read.  `host_weights[(layer, role)]`
    = (raw bytes, cols, rows, kind).  Returns one record per operator; raises AssertionError on the
    first operator outside its bound."""
    bf16 = chain.x_kind != 0
    records = []
    for op in ops:
        chain.issue(op)
        gpu.complete()
        cols, rows = op.w.t.dims[0], op.w.t.dims[1]
        a = gpu.read_f32(op.a, cols).copy()
        b = gpu.read_f32(op.b, cols).copy() if op.b is not None else None
        y = gpu.read_f32(op.y, rows).astype(np.float64)
        if op.w2 is None:
            raw, c, r, kind = host_weights[(op.layer, op.name)]
            s, e, tol = expect_projection(raw, c, r, kind, a, b, bf16)
        else:
            raw_g, c, r, kind = host_weights[(op.layer, "gate")]
            raw_u = host_weights[(op.layer, "up")][0]
            s, e, tol = expect_gate_up(raw_g, raw_u, c, r, kind, a, b, bf16, op.gelu)
        assert (c, r) == (cols, rows)
        err = np.abs(y - e)
        worst = int(np.argmax(err / tol))
        rec = {"op": op.name, "layer": op.layer, "rows": rows, "cols": cols, "max_err_over_tol": float(err[worst] / tol[worst]),
               "rms": float(np.sqrt(np.mean(e * e)))}
        records.append(rec)
        assert (err <= tol).all(), f"{op.name} of layer {op.layer}: row {worst} off by {err[worst]:.6g} (bound {tol[worst]:.6g}, expected {e[worst]:.6g})"
        if op.s is not None:
            got_s = gpu.read_f32(op.s, cols)
            assert np.array_equal(got_s.view(np.uint32), s.view(np.uint32)), f"{op.name} of layer {op.layer}: stored residual sum differs"
    return records


class OracleChain:
    """The same token step on the CPU: the weights of ingot_b200.chain.DecodeChain (same seeds) and
    the same operator order, every projection an oracle GEMV."""

    def __init__(self, shape, layers: int | None = None, seed: int = 0, bf16: bool = True):
        from ingot_b200 import synth
        from ingot_b200.chain import layer_roles, weight_seed
        self.shape, self.bf16 = shape, bf16
        self.n_layers = shape.layers if layers is None else layers
        self.w = {}
        for layer in range(self.n_layers):
            for role, cols, rows in layer_roles(shape):
                kind = shape.kinds[role]
                self.w[(layer, role)] = (synth.random_matrix(kind, cols, rows, seed=weight_seed(seed, layer, role)), cols, rows, kind)
        kind = shape.kinds["head"]
        self.w[(self.n_layers, "head")] = (synth.random_matrix(kind, shape.hidden, shape.vocab, seed=weight_seed(seed, self.n_layers, "head")),
                                           shape.hidden, shape.vocab, kind)
        self.bytes = sum(v[0].size for v in self.w.values())

    def _project(self, key, a, b, f64: bool, threads: int):
        raw, cols, rows, kind = self.w[key]
        s, x, _ = normalised_input(a, b, self.bf16)
        if f64:
            return s, O.matvec_f64(raw, cols, rows, kind, x.reshape(1, cols))[0].astype(np.float32)
        return s, O.matvec_f32(raw, cols, rows, kind, x.reshape(1, cols), threads=threads)[0]

    def step(self, h0: np.ndarray, f64: bool = True, threads: int = 1) -> np.ndarray:
        """Logits (float32 [vocab]) of one token whose input hidden state is h0 [hidden]."""
        cur, delta = np.ascontiguousarray(h0, np.float32).reshape(-1), None
        for layer in range(self.n_layers):
            _, k = self._project((layer, "k"), cur, delta, f64, threads)
            _, v = self._project((layer, "v"), cur, delta, f64, threads)
            s, q = self._project((layer, "q"), cur, delta, f64, threads)
            if delta is not None:
                cur = s
            _, o = self._project((layer, "o"), q, None, f64, threads)
            after, g = self._project((layer, "gate"), cur, o, f64, threads)
            _, u = self._project((layer, "up"), cur, o, f64, threads)
            act = O.glu(g, u, self.shape.gelu)
            cur = after
            _, delta = self._project((layer, "down"), act, None, f64, threads)
        return self._project((self.n_layers, "head"), cur, delta, f64, threads)[1]
