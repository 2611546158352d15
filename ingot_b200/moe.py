"""Expert-routed FFN of a MoE decoder at decode time, issued through the C ABI.

The data flow is the MoE branch of the reference's `Generic::ffn`
(src/generic.rs:508-574): router logits -> `route_topk` -> routed gate/up + SiLU
(`generic_routed_gate_up`) -> routed down projection with one input row per pair
(`generic_routed`, per_pair) -> `moe_sum` in route order.  Ids and weights never
leave the device.

Expert parallelism (not in the reference, which keeps all experts on one device):
rank r of n owns experts [r*E/n, (r+1)*E/n).  Every rank sees the same tokens and
routing; `ep_localize` keeps a rank's own pairs, the routed GEMVs write zero rows for
the others, `moe_sum` gives the rank's partial output and an all-reduce (the
`all_reduce` callback) completes it.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from . import synth
from .gpu import F32, Buffer, Gpu, Tensor, Weight


@dataclass
class MoeShape:
    name: str
    layers: int
    hidden: int
    experts: int
    top: int
    ffn: int
    kind: int


QWEN3_30B_A3B = MoeShape("qwen3-30b-a3b-q4_k", 48, 2048, 128, 8, 768, synth.Q4_K)


def expert_range(experts: int, rank: int, world: int) -> tuple[int, int]:
    """Experts [first, end) that `rank` owns out of `world`."""
    return experts * rank // world, experts * (rank + 1) // world


def expert_bytes(s: MoeShape) -> int:
    """Bytes of one expert's three matrices."""
    return 2 * synth.stride_of(s.kind, s.hidden) * s.ffn + synth.stride_of(s.kind, s.ffn) * s.hidden


class MoeChain:
    """`layers` MoE FFN layers (this rank's experts) resident in HBM and the buffers of one
    decode step for `tokens` tokens."""

    def __init__(self, gpu: Gpu, shape: MoeShape, tokens: int = 1, seed: int = 0, rank: int = 0, world: int = 1,
                 all_reduce=None, layers: int | None = None, keep_host: bool = False, local_weights_only: bool = False,
                 group=None):
        """world > 1 without `group`: every rank holds all `tokens` tokens, runs its experts' pairs and the partial
        sums are all-reduced.  With `group` (gpu.Group): `tokens` are this rank's OWN tokens; rows travel to the
        experts' owners and back (token all-to-all, ingot_ep_*)."""
        self.gpu, self.shape, self.tokens = gpu, shape, tokens
        self.rank, self.world, self.all_reduce = rank, world, all_reduce
        self.group = group if world > 1 else None
        self.n_layers = shape.layers if layers is None else layers
        gpu.set_option(5, world)                  # INGOT_OPT_EP_WORLD: routed launches expect pairs / world live pairs
        self.first, end = expert_range(shape.experts, rank, world)
        self.local = end - self.first
        self.host = []
        self.weights = []
        s = shape
        for layer in range(self.n_layers):
            mats = {}
            for i, (role, cols, rows) in enumerate((("gate", s.hidden, s.ffn), ("up", s.hidden, s.ffn),
                                                    ("down", s.ffn, s.hidden))):
                per = synth.stride_of(s.kind, cols) * rows
                if local_weights_only:      # throughput runs: draw only this rank's experts (not the same values for every world size)
                    raw = None
                    mine = synth.random_matrix(s.kind, cols, rows, self.local,
                                               seed=(seed * 7919 + layer * 8 + i + 1000003 * rank) & 0x7FFFFFFF)
                else:
                    raw = synth.random_matrix(s.kind, cols, rows, s.experts, seed=(seed * 7919 + layer * 8 + i) & 0x7FFFFFFF)
                    mine = raw[self.first * per:end * per]
                t = Tensor.of([cols, rows, self.local], s.kind)
                mats[role] = Weight(gpu.load_weight(mine, t), t)
                if keep_host:
                    mats[role + "_host"] = raw
            self.weights.append(mats)
        pairs = tokens * s.top
        self.x = gpu.zeros(tokens * s.hidden)                 # FFN input (float32, replicated on every rank)
        self.logits = gpu.zeros(tokens * s.experts)           # router logits (synthetic N(0,1) in the benchmark)
        self.ids = gpu.empty_bytes(4 * pairs)
        self.w = gpu.zeros(pairs)
        self.ids_l = gpu.empty_bytes(4 * pairs)
        self.w_l = gpu.zeros(pairs)
        self.act = gpu.zeros(pairs * s.ffn)
        self.out = gpu.zeros(pairs * s.hidden)
        self.y = gpu.zeros(tokens * s.hidden)
        # the expert grouping of the packed path (more than four tokens; Generic::moe_packed, src/generic.rs:578-660)
        self.blocks = (pairs + 31) // 32 + s.experts
        self.layout = gpu.empty_bytes(4 * 2 * s.experts)
        self.tiles = gpu.empty_bytes(4 * 4 * self.blocks)
        self.packed = gpu.empty_bytes(4 * pairs)
        self.inverse = gpu.empty_bytes(4 * pairs)
        self.grouped = True           # tokens > 4 take the grouped path on one device; False: pair by pair (comparison)
        self.gemm_tokens = 256        # more tokens than this: per-expert tensor-core GEMMs over the packed rows (prefill width)
        self.x_packed = gpu.zeros(pairs * s.hidden) if tokens > self.gemm_tokens else None
        # token all-to-all: the received places run pair by pair unless this is set (with a few places per expert and
        # rank the grouped kernel measured slower on two GPUs: 13.4 against 11.8 ms per 32-token step)
        self.grouped_places = False
        self.launches_per_step = 0
        if self.group:
            from .gpu import EpExchange
            self.cap = pairs                                  # places per sending rank: all its pairs may choose one owner
            self.ep = EpExchange(self.group, self.cap, s.hidden)
            places = world * self.cap
            self.ids_rx = gpu.empty_bytes(4 * places)
            self.act_rx = gpu.zeros(places * s.ffn)
            self.out_rx = gpu.zeros(places * s.hidden)
            self.tiles_rx = gpu.empty_bytes(4 * 4 * ((places + 31) // 32 + self.local))
            self.packed_rx = gpu.empty_bytes(4 * places)
            self.inverse_rx = gpu.empty_bytes(4 * places)

    def set_capacity(self, cap: int) -> None:
        """Places per sending rank for the next steps (the same on every rank, at most what the areas were sized
        for): the routed projections run over world x cap places, so a tight capacity keeps their grids small."""
        if cap * self.shape.hidden > self.ep.ret_rows.nbytes // 4:
            raise ValueError("capacity beyond the exchange areas")
        self.cap = self.ep.cap = cap

    @staticmethod
    def exchange_slots(layers: int) -> int:
        """Slots a group needs for the token all-to-all: dispatch and return of every layer."""
        return 2 * layers

    def layer(self, i: int) -> None:
        """One MoE FFN layer on the handle's stream: y = sum_k w_k * down_k(silu(gate_k x) * up_k x)."""
        g, s, lib, h = self.gpu, self.shape, self.gpu._lib, self.gpu._h
        pairs = self.tokens * s.top
        ws = self.weights[i]
        g._check(lib.ingot_route_topk(h, self.logits.ptr, s.experts, s.top, self.tokens, self.ids.ptr, self.w.ptr))
        ids, w = self.ids, self.w
        n = 1
        if self.group:
            # token all-to-all: this rank's pairs go to the experts' owners; the places received from all ranks are
            # run pair by pair (one activation row per place), their rows go home and are summed there
            ep, places = self.ep, self.world * self.cap
            ep.dispatch(2 * i, self.x, self.ids, self.tokens, s.top, self.local)
            ep.receive(2 * i, self.ids_rx)
            tg, td = ws["gate"].t, ws["down"].t
            if self.grouped_places and places > 4:
                # the places of one expert share its rows: grouped by expert, four at a time (skipped places take no position)
                blocks = (places + 31) // 32 + self.local
                g._check(lib.ingot_expert_layout(h, self.ids_rx.ptr, places, self.local, blocks, self.layout.ptr, self.tiles_rx.ptr,
                                                 self.packed_rx.ptr, self.inverse_rx.ptr))
                g._check(lib.ingot_expert_gate_up(h, ws["gate"].buffer.ptr, ws["up"].buffer.ptr, tg.dims[0], tg.dims[1], tg.stride, tg.kind,
                                                  self.local, ep.rx_rows.ptr, self.tiles_rx.ptr, self.packed_rx.ptr, blocks, 1, places,
                                                  self.act_rx.ptr))
                g._check(lib.ingot_expert_project(h, ws["down"].buffer.ptr, td.dims[0], td.dims[1], td.stride, td.kind, self.local,
                                                  self.act_rx.ptr, self.tiles_rx.ptr, self.packed_rx.ptr, blocks, 1, places, 0, self.out_rx.ptr))
                ep.give_back(2 * i + 1, self.out_rx, self.inverse_rx)
                ep.combine(2 * i + 1, self.w, s.top, self.tokens, self.y)
                self.launches_per_step += 8
                return
            g._check(lib.ingot_routed_gate_up(h, ws["gate"].buffer.ptr, ws["up"].buffer.ptr, tg.dims[0], tg.dims[1], tg.stride,
                                              tg.kind, self.local, ep.rx_rows.ptr, F32, self.ids_rx.ptr, 1, places, self.act_rx.ptr))
            g._check(lib.ingot_routed(h, ws["down"].buffer.ptr, td.dims[0], td.dims[1], td.stride, td.kind, self.local,
                                      self.act_rx.ptr, F32, self.ids_rx.ptr, 1, 1, places, self.out_rx.ptr))
            ep.give_back(2 * i + 1, self.out_rx)
            ep.combine(2 * i + 1, self.w, s.top, self.tokens, self.y)
            self.launches_per_step += 7
            return
        if self.world > 1:
            g._check(lib.ingot_ep_localize(h, self.ids.ptr, self.w.ptr, pairs, self.first, self.local, self.ids_l.ptr,
                                           self.w_l.ptr))
            ids, w = self.ids_l, self.w_l
            n += 1
        tg, td = ws["gate"].t, ws["down"].t
        if self.tokens > self.gemm_tokens and self.world == 1 and self.grouped:
            # prefill width: the rows in packed order, then every expert's run of rows through the tensor-core GEMM
            blocks = (pairs + 31) // 32 + s.experts
            g._check(lib.ingot_expert_layout(h, ids.ptr, pairs, s.experts, blocks, self.layout.ptr, self.tiles.ptr, self.packed.ptr,
                                             self.inverse.ptr))
            g._check(lib.ingot_gather_rows(h, self.x.ptr, self.packed.ptr, pairs, s.top, s.hidden, self.x_packed.ptr))
            g._check(lib.ingot_expert_gemm_gate_up(h, ws["gate"].buffer.ptr, ws["up"].buffer.ptr, tg.dims[0], tg.dims[1], tg.stride, tg.kind,
                                                   self.local, self.x_packed.ptr, self.layout.ptr, pairs, 0, self.act.ptr))
            g._check(lib.ingot_expert_gemm(h, ws["down"].buffer.ptr, td.dims[0], td.dims[1], td.stride, td.kind, self.local,
                                           self.act.ptr, self.layout.ptr, pairs, self.out.ptr))
            g._check(lib.ingot_combine_packed(h, self.out.ptr, w.ptr, self.inverse.ptr, s.hidden, s.top, self.tokens, self.y.ptr))
            return
        if self.tokens > 4 and self.world == 1 and self.grouped:
            # every expert touched is streamed once per four of its pairs, not once per pair
            blocks = (pairs + 31) // 32 + s.experts
            g._check(lib.ingot_expert_layout(h, ids.ptr, pairs, s.experts, blocks, self.layout.ptr, self.tiles.ptr, self.packed.ptr,
                                             self.inverse.ptr))
            g._check(lib.ingot_expert_gate_up(h, ws["gate"].buffer.ptr, ws["up"].buffer.ptr, tg.dims[0], tg.dims[1], tg.stride, tg.kind,
                                              self.local, self.x.ptr, self.tiles.ptr, self.packed.ptr, blocks, s.top, pairs, self.act.ptr))
            g._check(lib.ingot_expert_project(h, ws["down"].buffer.ptr, td.dims[0], td.dims[1], td.stride, td.kind, self.local,
                                              self.act.ptr, self.tiles.ptr, self.packed.ptr, blocks, s.top, pairs, 0, self.out.ptr))
            g._check(lib.ingot_combine_packed(h, self.out.ptr, w.ptr, self.inverse.ptr, s.hidden, s.top, self.tokens, self.y.ptr))
            self.launches_per_step += 5
            return
        g._check(lib.ingot_routed_gate_up(h, ws["gate"].buffer.ptr, ws["up"].buffer.ptr, tg.dims[0], tg.dims[1], tg.stride,
                                          tg.kind, self.local, self.x.ptr, F32, ids.ptr, s.top, pairs, self.act.ptr))
        g._check(lib.ingot_routed(h, ws["down"].buffer.ptr, td.dims[0], td.dims[1], td.stride, td.kind, self.local,
                                  self.act.ptr, F32, ids.ptr, 1, s.top, pairs, self.out.ptr))
        g._check(lib.ingot_moe_sum(h, self.out.ptr, w.ptr, s.hidden, s.top, self.tokens, self.y.ptr))
        self.launches_per_step += n + 3
        if self.world > 1:
            self.all_reduce(self.y, self.tokens * s.hidden)

    def step(self) -> None:
        self.launches_per_step = 0
        if self.group:
            self.group.step()
            self.launches_per_step += 1
        for i in range(self.n_layers):
            self.layer(i)

    def record(self):
        self.gpu.record()
        self.step()
        return self.gpu.end_record()

    def unique_expert_bytes(self, ids: np.ndarray) -> int:
        """Algorithmic weight bytes of one layer for routing `ids`: unique experts x 3 matrices."""
        return len(np.unique(ids)) * expert_bytes(self.shape)
