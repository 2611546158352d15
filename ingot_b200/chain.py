"""The per-token GEMV chain of a dense decoder, issued through the C ABI.

This is the projection skeleton of the reference's `Generic::hidden`
(src/generic.rs:664-763) at decode: per layer q, k, v, o, fused gate/up + GLU,
down; then the output head.  Attention itself is not on this path: the
attention output is stood in for by the (normalised) q projection so that every
weight byte of a token step is still streamed exactly once and magnitudes stay
O(1) through the layers.  Between projections an unweighted RMS normalisation
(`add_rms`, kernels/generic.metal:390-404) carries the residual stream in
float32 and hands bfloat16 (or float32) activations to the next projection.

Rows can be sharded tensor-parallel: rank r of n owns rows [r*N/n, (r+1)*N/n) of
every matrix (block quantisation runs along K, so a row split keeps the GGUF
layout) and an `all_gather` callback rebuilds full activations where the next
operator needs them.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from . import synth
from .gpu import BF16, F32, X_PACKED, X_PACKED_HI, Buffer, Gpu, Tensor, Weight


@dataclass
class DenseShape:
    name: str
    layers: int
    hidden: int
    q: int            # rows of the q projection (= o's cols)
    kv: int
    ffn: int
    vocab: int
    kinds: dict       # role -> GGML kind
    gelu: bool = False


@dataclass
class FusedOp:
    """One projection of the fused step together with the add_rms it consumes."""
    name: str
    layer: int
    w: Weight
    w2: Weight | None      # the up matrix of a fused gate/up
    a: Buffer
    b: Buffer | None
    s: Buffer | None
    y: Buffer
    scope: int | None = None
    shard_only: bool = False      # row shards: nobody reads the whole vector, the shard stays at the front of y
    gather_late: bool = False     # row shards: gathered after the operator's scope has closed
    gelu: bool = False
    signal: int | None = None     # row shards with a group: the exchange slot this operator's rows raise on every rank
    waits: tuple = ()             # ... and the slots of the assembled inputs it waits for


QWEN3_8B = DenseShape("qwen3-8b-q4_k_m", 36, 4096, 4096, 1024, 12288, 151936,
                      {"q": synth.Q4_K, "k": synth.Q4_K, "v": synth.Q6_K, "o": synth.Q4_K, "gate": synth.Q4_K,
                       "up": synth.Q4_K, "down": synth.Q6_K, "head": synth.Q6_K})
GEMMA3_4B = DenseShape("gemma3-4b-q4_0", 34, 2560, 2048, 1024, 10240, 262144,
                       {r: synth.Q4_0 for r in ("q", "k", "v", "o", "gate", "up", "down", "head")}, gelu=True)


def layer_roles(s: DenseShape):
    """(role, cols, rows) of one layer."""
    return [("q", s.hidden, s.q), ("k", s.hidden, s.kv), ("v", s.hidden, s.kv), ("o", s.q, s.hidden),
            ("gate", s.hidden, s.ffn), ("up", s.hidden, s.ffn), ("down", s.ffn, s.hidden)]


def weight_bytes_per_token(s: DenseShape) -> int:
    per_layer = sum(synth.stride_of(s.kinds[r], c) * n for r, c, n in layer_roles(s))
    return s.layers * per_layer + synth.stride_of(s.kinds["head"], s.hidden) * s.vocab


def weight_seed(seed: int, layer: int, role: str) -> int:
    """Seed of the synthetic matrix of `role` in `layer` (the head counts as layer `n_layers`)."""
    role_id = ["q", "k", "v", "o", "gate", "up", "down", "head"].index(role)
    return (seed * 1000003 + layer * 64 + role_id) & 0x7FFFFFFF


def shard_rows(rows: int, rank: int, world: int) -> tuple[int, int]:
    """Rows [begin, end) that `rank` owns out of `world`."""
    return rows * rank // world, rows * (rank + 1) // world


class _null_scope:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


class DecodeChain:
    """Weights of one dense model (or this rank's row shard) resident in HBM and the
    buffers of one decode step for `batch` tokens."""

    def __init__(self, gpu: Gpu, shape: DenseShape, batch: int = 1, x_kind: int = BF16, seed: int = 0,
                 rank: int = 0, world: int = 1, all_gather=None, layers: int | None = None,
                 keep_host: int = 0, packed: bool = True, independent_qkv: bool = True, fused_norm: bool = True, group=None):
        self.gpu, self.shape, self.batch, self.x_kind = gpu, shape, batch, x_kind
        self.rank, self.world, self.all_gather = rank, world, all_gather
        # a tensor-parallel group (gpu.Group): the projections exchange their row shards themselves (peer stores and
        # arrival counters) instead of an all-gather after each of them
        self.group = group if world > 1 else None
        self.n_layers = shape.layers if layers is None else layers
        self.host = {}                 # (layer, role) -> (bytes, cols, rows, kind) kept for checks/baselines
        self.weights: list[dict[str, Weight]] = []
        self.bytes_streamed = 0
        for layer in range(self.n_layers):
            ws = {}
            for role, cols, rows in layer_roles(shape):
                ws[role] = self._make(layer, role, cols, rows, shape.kinds[role], seed, layer < keep_host)
            self.weights.append(ws)
        self.head = self._make(self.n_layers, "head", shape.hidden, shape.vocab, shape.kinds["head"], seed,
                               keep_host > 0)
        b, h = batch, shape.hidden
        xb = 2 if x_kind == BF16 else 4
        self.h_in = gpu.zeros(b * h)                  # the step's input hidden state (float32)
        self.h = gpu.zeros(b * h)                     # residual stream
        self.xn = gpu.empty_bytes(b * h * xb)
        shared = self.group.alloc if self.group else gpu.zeros        # vectors every rank needs whole live in the group's window
        self.q, self.k, self.v = shared(b * shape.q), gpu.zeros(b * shape.kv), gpu.zeros(b * shape.kv)
        self.a = gpu.empty_bytes(b * shape.q * xb)
        self.o = shared(b * h)
        self.act = shared(b * shape.ffn)
        self.actn = gpu.empty_bytes(b * shape.ffn * xb)
        self.d = shared(b * h)
        self.logits = shared(b * shape.vocab)
        # per-rank partial outputs when sharded
        self.part = gpu.zeros(b * max(shape.ffn, shape.vocab) // world + b * 8) if world > 1 else None
        # activations packed once per distinct GEMV input (one token: the tensor-core GEMV)
        self.packed = batch == 1 and packed
        # several tokens: bfloat16 activations as high-part rows, eight tokens per pass over the weights
        self.packed_hi = (batch > 1 and packed and x_kind == BF16 and world == 1
                          and all(k in (synth.Q4_K, synth.Q6_K) for k in shape.kinds.values())
                          and all(c % 2048 == 0 for _, c, _ in layer_roles(shape)))
        # add_rms fused into the projections that consume it (one token, tensor-core GEMV kinds only)
        tc_kinds = (synth.Q4_0, synth.Q8_0, synth.Q4_K, synth.Q6_K)
        self.fused_norm = (fused_norm and self.packed and all(k in tc_kinds for k in shape.kinds.values())
                           and all(synth.stride_of(shape.kinds[r], c) % 16 == 0 for r, c, _ in layer_roles(shape)))
        # q, k and v read the same activations and write different buffers: issue them concurrently
        # (the reference's independent_projections scope); row shards: only the fused step, which gathers q after the scope
        self.independent_qkv = independent_qkv and self.packed and (world == 1 or self.fused_norm)
        # ... and the scope launches them as one grid when all three take the tensor-core GEMV
        self.grouped_qkv = self.independent_qkv and all(
            shape.kinds[r] in (synth.Q4_0, synth.Q8_0, synth.Q4_K, synth.Q6_K) and shape.hidden % 64 == 0
            and synth.stride_of(shape.kinds[r], shape.hidden) % 16 == 0 for r in ("q", "k", "v"))
        self.h2 = gpu.zeros(b * h) if self.fused_norm else None        # the residual stream alternates between h and h2
        if self.packed or self.packed_hi:
            size = (lambda c: batch * gpu.packed_hi_bytes(c)) if self.packed_hi else gpu.packed_x_bytes
            self.xn_p = gpu.empty_bytes(size(h))
            self.a_p = gpu.empty_bytes(size(shape.q))
            self.actn_p = gpu.empty_bytes(size(shape.ffn))
        self.launches_per_step = 0

    def _make(self, layer, role, cols, rows, kind, seed, keep) -> Weight:
        r0, r1 = shard_rows(rows, self.rank, self.world)
        stride = synth.stride_of(kind, cols)
        full_seed = weight_seed(seed, layer, role)
        if self.world == 1:
            raw = synth.random_matrix(kind, cols, rows, seed=full_seed)
        else:   # every rank draws the same full matrix stream and keeps its rows
            raw = synth.random_matrix(kind, cols, rows, seed=full_seed).reshape(rows, stride)[r0:r1].reshape(-1)
        if keep:
            self.host[(layer, role)] = (raw, cols, r1 - r0, kind)
        self.bytes_streamed += raw.size
        return Weight(self.gpu.load_weight(raw, Tensor.of([cols, r1 - r0], kind)), Tensor.of([cols, r1 - r0], kind))

    # ---- one decode step -------------------------------------------------------
    def _norm(self, a: Buffer, b: Buffer | None, s: Buffer | None, out: Buffer, width: int) -> None:
        g = self.gpu
        y32 = out.ptr if self.x_kind == F32 else None
        y16 = out.ptr if self.x_kind == BF16 else None
        packed = None
        if self.packed or self.packed_hi:
            packed = {self.xn.ptr: self.xn_p, self.a.ptr: self.a_p, self.actn.ptr: self.actn_p}[out.ptr].ptr
        mode = 3 if self.packed_hi else int(self.x_kind == BF16)
        g._check(g._lib.ingot_add_rms_packed(g._h, a.ptr, b.ptr if b else None, None, s.ptr if s else None, y32, y16,
                                             packed, mode, width, self.batch, 1e-6, 1 if b else 0))
        self.launches_per_step += 1

    def _x(self, x: Buffer):
        """(pointer, x_kind) of a GEMV input: the packed copy when there is one."""
        if self.packed or self.packed_hi:
            p = {self.xn.ptr: self.xn_p, self.a.ptr: self.a_p, self.actn.ptr: self.actn_p}[x.ptr].ptr
            return p, (X_PACKED_HI if self.packed_hi else X_PACKED)
        return x.ptr, self.x_kind

    def _project(self, w: Weight, x: Buffer, y: Buffer) -> None:
        g, t = self.gpu, w.t
        dst = y if self.world == 1 else self.part
        xp, xk = self._x(x)
        g._check(g._lib.ingot_matmul(g._h, w.buffer.ptr, t.dims[0], t.dims[1], t.stride, t.kind, 0, xp, xk, self.batch,
                                     dst.ptr))
        self.launches_per_step += 1
        if self.world > 1:
            self.all_gather(dst, y, self.batch, t.dims[1])

    def _gate_up(self, gate: Weight, up: Weight, x: Buffer, y: Buffer) -> None:
        g, t = self.gpu, gate.t
        dst = y if self.world == 1 else self.part
        xp, xk = self._x(x)
        g._check(g._lib.ingot_gate_up(g._h, gate.buffer.ptr, up.buffer.ptr, t.dims[0], t.dims[1], t.stride, t.kind,
                                      xp, xk, self.batch, int(self.shape.gelu), dst.ptr))
        self.launches_per_step += 1
        if self.world > 1:
            self.all_gather(dst, y, self.batch, t.dims[1])

    # ---- the same step with every add_rms fused into its consumers ------------------------
    def fused_ops(self) -> list["FusedOp"]:
        """The fused step as a list of operators in issue order: every projection with the add_rms it
        consumes (`y = w . rms_norm(a + b)`, the sum stored to `s`).  Operators that share a `scope`
        number are independent of each other and are issued inside one independent scope."""
        s = self.shape
        ops: list[FusedOp] = []
        cur, delta = self.h_in, None            # residual stream so far and the update not yet added to it
        bufs = [self.h, self.h2]
        nxt = 0
        for li, ws in enumerate(self.weights):
            # q, k, v read rms_norm(cur + delta); q also stores the sum
            summed = bufs[nxt] if delta else None
            scope = li if self.independent_qkv else None
            # the two small projections first: their CTAs leave room for q's to start beside them
            # (attention over row-sharded k and v is local to a rank's heads: they are never gathered)
            ops.append(FusedOp("k", li, ws["k"], None, cur, delta, None, self.k, scope=scope, shard_only=True))
            ops.append(FusedOp("v", li, ws["v"], None, cur, delta, None, self.v, scope=scope, shard_only=True))
            ops.append(FusedOp("q", li, ws["q"], None, cur, delta, summed, self.q, scope=scope, gather_late=True))
            if delta:
                cur, nxt = summed, nxt ^ 1
            ops.append(FusedOp("o", li, ws["o"], None, self.q, None, None, self.o))      # stands in for attention: o(rms_norm(q))
            after = bufs[nxt]
            ops.append(FusedOp("gate_up", li, ws["gate"], ws["up"], cur, self.o, after, self.act, gelu=s.gelu))
            cur, nxt = after, nxt ^ 1
            ops.append(FusedOp("down", li, ws["down"], None, self.act, None, None, self.d))
            delta = self.d
        ops.append(FusedOp("head", self.n_layers, self.head, None, cur, delta, None, self.logits))
        if self.group:
            # one exchange slot per operator whose rows every rank needs; an operator waits for the slots of the
            # vectors among its inputs that were assembled that way (the latest writer of each)
            slot_of: dict[int, int] = {}
            n = 0
            for op in ops:
                op.waits = tuple(slot_of[x.ptr] for x in (op.a, op.b) if x is not None and x.ptr in slot_of)
                if not op.shard_only:
                    op.signal, n = n, n + 1
                    slot_of[op.y.ptr] = op.signal
        return ops

    @staticmethod
    def exchange_slots(layers: int) -> int:
        """Slots a group needs for this chain: q, o, gate/up and down of every layer, and the head."""
        return 4 * layers + 1

    def issue(self, op: "FusedOp") -> None:
        """Issues one fused operator (and, on a row shard, the gather of its result)."""
        g, t = self.gpu, op.w.t
        sharded = self.world > 1 and not op.shard_only
        dst = self.part if sharded else op.y           # every rank norms the whole input itself
        if self.group:
            # the rows go straight to their place in the whole vector, here and on every peer
            r0, _ = shard_rows(self._full_rows(op), self.rank, self.world)
            dst = op.y if op.shard_only else op.y.view_f32(r0, t.dims[1])
            if op.signal is not None:
                self.group.signal_next(op.signal)
            if op.waits:
                self.group.wait_next(*op.waits)
        a, b, sm = op.a.ptr, op.b.ptr if op.b else None, op.s.ptr if op.s else None
        rb = int(self.x_kind == BF16)
        if op.w2 is None:
            g._check(g._lib.ingot_matmul_normed(g._h, op.w.buffer.ptr, t.dims[0], t.dims[1], t.stride, t.kind, 0, a, b, None,
                                                sm, 1e-6, 1 if op.b else 0, rb, dst.ptr))
        else:
            g._check(g._lib.ingot_gate_up_normed(g._h, op.w.buffer.ptr, op.w2.buffer.ptr, t.dims[0], t.dims[1], t.stride,
                                                 t.kind, a, b, None, sm, 1e-6, 1 if op.b else 0, rb, int(op.gelu), dst.ptr))
        self.launches_per_step += 1
        if sharded and not op.gather_late and not self.group:
            self.all_gather(dst, op.y, self.batch, t.dims[1])

    def _full_rows(self, op: "FusedOp") -> int:
        """Rows of the operator's whole (unsharded) output."""
        s = self.shape
        return {"q": s.q, "k": s.kv, "v": s.kv, "o": s.hidden, "gate_up": s.ffn, "down": s.hidden, "head": s.vocab}[op.name]

    def _step_fused(self) -> None:
        g = self.gpu
        self.launches_per_step = 0
        if self.group:
            self.group.step()
            self.launches_per_step += 1
        ops = self.fused_ops()
        i = 0
        while i < len(ops):
            j = i + 1
            if ops[i].scope is not None:
                while j < len(ops) and ops[j].scope == ops[i].scope:
                    j += 1
            with g.independent() if j - i > 1 else _null_scope():
                for op in ops[i:j]:
                    self.issue(op)
            for op in ops[i:j]:
                if self.world > 1 and op.gather_late and not op.shard_only and not self.group:
                    self.all_gather(self.part, op.y, self.batch, op.w.t.dims[1])
            if j - i > 1:
                self.launches_per_step -= j - i - 1      # the scope issues its projections as one grid
            i = j
        if self.group:
            self.group.wait(ops[-1].signal, ops[-1].y)   # the logits of every rank, for whoever reads them after the step
            self.launches_per_step += 1

    def step(self) -> None:
        """Issues one token step on the handle's stream (asynchronous)."""
        if self.fused_norm:
            return self._step_fused()
        s = self.shape
        self.launches_per_step = 0
        delta = None
        src = self.h_in
        for ws in self.weights:
            self._norm(src, delta, self.h if delta else None, self.xn, s.hidden)
            if delta is None and src is self.h_in:
                resid = self.h_in
            else:
                resid = self.h
            if self.independent_qkv:
                with self.gpu.independent():
                    self._project(ws["q"], self.xn, self.q)
                    self._project(ws["k"], self.xn, self.k)
                    self._project(ws["v"], self.xn, self.v)
                if self.grouped_qkv:
                    self.launches_per_step -= 2      # the scope issues its three projections as one grid
            else:
                self._project(ws["q"], self.xn, self.q)
                self._project(ws["k"], self.xn, self.k)
                self._project(ws["v"], self.xn, self.v)
            self._norm(self.q, None, None, self.a, s.q)
            self._project(ws["o"], self.a, self.o)
            self._norm(resid, self.o, self.h, self.xn, s.hidden)
            self._gate_up(ws["gate"], ws["up"], self.xn, self.act)
            self._norm(self.act, None, None, self.actn, s.ffn)
            self._project(ws["down"], self.actn, self.d)
            src, delta = self.h, self.d
        self._norm(src, delta, self.h if delta else None, self.xn, s.hidden)
        self._project(self.head, self.xn, self.logits)

    def record_chain(self):
        """Records the fused step as a chain: one persistent kernel per token step."""
        if not self.fused_norm or self.world != 1:
            raise ValueError("only the fused one-token step of a single device can be recorded as a chain")
        self.gpu.chain_begin()
        try:
            self.step()
        except Exception:
            try:
                self.gpu.chain_end()
            except Exception:
                pass
            raise
        self.launches_per_step = 1
        return self.gpu.chain_end()

    def record(self):
        """Records one step as a replayable command (a CUDA graph)."""
        self.gpu.record()
        self.step()
        return self.gpu.end_record()
