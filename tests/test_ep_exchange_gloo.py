"""The expert-parallel token all-to-all on CPU: two `gloo` ranks hold their own tokens, route them, exchange
rows by the bookkeeping the device kernels implement (oracle/ep_exchange.py restates it), run their experts with
the oracle, send the rows home and sum them there.  Every token's result must equal the single-rank layer."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ingot_b200 import synth
from oracle import ep_exchange as X
from oracle import oracle as O


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _gather(t: torch.Tensor, world: int) -> list:
    out = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(out, t)
    return out


def _worker(rank: int, world: int, port: int, out_dir: str):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        kind = synth.Q4_K
        experts, hidden, ffn, top, tokens = 8, 256, 256, 3, 3            # tokens per rank
        epr, cap = experts // world, tokens * top
        g, u = synth.random_matrix(kind, hidden, ffn, experts, 1), synth.random_matrix(kind, hidden, ffn, experts, 2)
        d = synth.random_matrix(kind, ffn, hidden, experts, 3)
        logits = np.random.default_rng(10 + rank).normal(0, 1, (tokens, experts)).astype(np.float32)
        xs = synth.activations(tokens, hidden, seed=20 + rank) * np.float32(0.05)
        routed = [O.route(logits[t], top) for t in range(tokens)]
        ids = np.concatenate([r[0] for r in routed]).astype(np.uint32)
        wts = np.concatenate([r[1] for r in routed]).astype(np.float32)

        def ffn_out(x, e):
            a = O.glu(O.matvec_f64(g, hidden, ffn, kind, x, expert=e)[0].astype(np.float32),
                      O.matvec_f64(u, hidden, ffn, kind, x, expert=e)[0].astype(np.float32))
            return O.matvec_f64(d, ffn, hidden, kind, a, expert=e)[0].astype(np.float32)

        # dispatch: rows and words into region `rank` of every owner (here: everything is gathered, each owner picks)
        owner, place, meta = X.dispatch_plan(ids, world, epr, cap)
        rows = np.zeros((world, cap, hidden), dtype=np.float32)
        for p in range(len(ids)):
            rows[owner[p], place[p]] = xs[p // top]
        all_meta = [m.numpy().view(np.uint32) for m in _gather(torch.from_numpy(meta.view(np.int32).copy()), world)]
        all_rows = [r.numpy() for r in _gather(torch.from_numpy(rows), world)]
        # receive: region s = what rank s sent to this owner
        region, ids_rx = X.receive_regions(all_meta, rank)
        rx_rows = np.concatenate([all_rows[s][rank] for s in range(world)])
        out_rx = np.zeros((world * cap, hidden), dtype=np.float32)
        for i, e in enumerate(ids_rx):
            if e != X.ROUTE_SKIP:
                out_rx[i] = ffn_out(rx_rows[i], rank * epr + int(e))
        # return: every live place's row to its home rank at the pair's index
        back = np.zeros((world, cap, hidden), dtype=np.float32)
        for i, home, pair in X.way_home(region, cap):
            back[home, pair] = out_rx[i]
        got_back = [b.numpy() for b in _gather(torch.from_numpy(back), world)]
        ret_rows = sum(got_back[s][rank] for s in range(world))          # every pair comes from exactly one owner
        y = O.moe_sum(ret_rows[:tokens * top].reshape(-1), wts, hidden, top).reshape(tokens, hidden)
        # the single-rank layer on the same tokens
        want_rows = np.stack([ffn_out(xs[p // top], int(ids[p])) for p in range(len(ids))])
        want = O.moe_sum(want_rows.reshape(-1), wts, hidden, top).reshape(tokens, hidden)
        assert np.array_equal(y.view(np.uint32), want.view(np.uint32))
        # bookkeeping invariants: each pair has exactly one place, places of a region are dense from 0
        assert sorted((o, pl) for o, pl in zip(owner, place)) == [(o, k) for o in range(world) for k in range(int((owner == o).sum()))]
        open(os.path.join(out_dir, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


def test_token_all_to_all_with_two_gloo_ranks(tmp_path):
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert sorted(os.listdir(tmp_path)) == ["ok0", "ok1"]


def test_plan_edge_cases():
    # all pairs on one owner; no pairs at all; capacity exactly met
    owner, place, meta = X.dispatch_plan([5, 4, 7, 6], world=2, experts_per_rank=4, cap=4)
    assert list(owner) == [1, 1, 1, 1] and list(place) == [0, 1, 2, 3]
    assert (meta[0] == X.ROUTE_SKIP).all() and list(meta[1] & 0xFFFF) == [1, 0, 3, 2] and list(meta[1] >> 16) == [0, 1, 2, 3]
    owner, place, meta = X.dispatch_plan([], world=4, experts_per_rank=2, cap=3)
    assert len(owner) == 0 and (meta == X.ROUTE_SKIP).all()
    region, ids = X.receive_regions([meta, meta, meta, meta], 2)
    assert len(region) == 12 and (ids == X.ROUTE_SKIP).all() and X.way_home(region, 3) == []
