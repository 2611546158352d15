"""The multi-GPU partitioning logic on CPU: two `gloo` ranks shard a dense projection by
output rows (all-gather) and an MoE layer by experts (all-reduce of partial sums), with the
oracle doing the arithmetic, and must reproduce the single-rank result."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ingot_b200 import synth
from ingot_b200.chain import shard_rows
from ingot_b200.moe import expert_range
from oracle import oracle as O


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, out_dir: str):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # ---- dense: rows sharded, outputs all-gathered ----
        cols, rows, kind = 1024, 96, synth.Q4_K
        raw = synth.random_matrix(kind, cols, rows, seed=5)
        x = synth.activations(1, cols, seed=6)
        r0, r1 = shard_rows(rows, rank, world)
        stride = synth.stride_of(kind, cols)
        mine = raw.reshape(rows, stride)[r0:r1].reshape(-1)
        part = torch.from_numpy(O.matvec_f64(mine, cols, r1 - r0, kind, x)[0].copy())
        full = torch.empty(rows, dtype=torch.float64)
        dist.all_gather_into_tensor(full, part)
        want = O.matvec_f64(raw, cols, rows, kind, x)[0]
        assert np.array_equal(full.numpy(), want)
        # ---- MoE: experts sharded, partial sums all-reduced ----
        experts, hidden, ffn, top, tokens = 8, 256, 256, 3, 2
        g, u = synth.random_matrix(kind, hidden, ffn, experts, 1), synth.random_matrix(kind, hidden, ffn, experts, 2)
        d = synth.random_matrix(kind, ffn, hidden, experts, 3)
        logits = np.random.default_rng(0).normal(0, 1, (tokens, experts)).astype(np.float32)
        xs = synth.activations(tokens, hidden, seed=4) * np.float32(0.05)
        first, end = expert_range(experts, rank, world)

        def ffn_out(tok, e):
            a = O.glu(O.matvec_f64(g, hidden, ffn, kind, xs[tok], expert=e)[0].astype(np.float32),
                      O.matvec_f64(u, hidden, ffn, kind, xs[tok], expert=e)[0].astype(np.float32))
            return O.matvec_f64(d, ffn, hidden, kind, a, expert=e)[0]

        partial = np.zeros((tokens, hidden))
        total = np.zeros((tokens, hidden))
        for t in range(tokens):
            ids, w = O.route(logits[t], top)
            for e, wt in zip(ids, w):
                y = ffn_out(t, int(e)) * float(wt)
                total[t] += y
                if first <= e < end:
                    partial[t] += y
        red = torch.from_numpy(partial.copy())
        dist.all_reduce(red)
        assert np.allclose(red.numpy(), total, rtol=1e-12, atol=1e-12)
        open(os.path.join(out_dir, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


def test_row_and_expert_sharding_with_two_gloo_ranks(tmp_path):
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert sorted(os.listdir(tmp_path)) == ["ok0", "ok1"]


def test_shard_helpers_cover_everything_once():
    for n, world in ((4096, 8), (151936, 8), (1024, 4), (7, 2), (128, 8)):
        spans = [shard_rows(n, r, world) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        assert [expert_range(n, r, world) for r in range(world)] == spans
