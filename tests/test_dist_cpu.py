"""The multi-GPU plan of the path on CPU ranks (gloo, world_size 2): the
block-cyclic KV-sequence split partitions every position once, each rank's
partial over its own rows all-gathered as one [o | m | l] buffer merges to the
unsplit result, appends go to the owner of the position, and the GatedDeltaNet
sequences are dealt round-robin without overlap.  The arithmetic is the
oracle's; the split arithmetic is the library's host-side code."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import moeflux_b200 as M
import oracle as O
from oracle import A17B as G
from tests import inputs as I

WORLD = 2
BLOCK = 32


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, port, ctx_len, n_steps, result_path):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=WORLD)
    L = M.lib()
    r = I.rng(600)  # same stream on every rank: the ranks hold shares of the same sequence
    K, V = I.normal(r, (ctx_len + n_steps, G.kv_dim)), I.normal(r, (ctx_len + n_steps, G.kv_dim))
    H, D = G.num_attn_heads, G.head_dim
    # this rank's compact local cache, filled by ownership
    rows = [p for p in range(ctx_len) if L.mfc_kv_local_row(p, rank, WORLD, BLOCK) >= 0]
    assert [L.mfc_kv_local_row(p, rank, WORLD, BLOCK) for p in rows] == list(range(len(rows)))
    assert len(rows) == L.mfc_kv_local_len(ctx_len, rank, WORLD, BLOCK)
    Kl, Vl = list(K[rows]), list(V[rows])
    worst = 0.0
    for step in range(n_steps):
        pos = ctx_len + step
        q, gate = I.normal(r, G.q_dim), I.normal(r, G.q_dim)
        if L.mfc_kv_local_row(pos, rank, WORLD, BLOCK) >= 0:  # the owner appends
            assert L.mfc_kv_local_row(pos, rank, WORLD, BLOCK) == len(Kl)
            Kl.append(K[pos])
            Vl.append(V[pos])
        n_loc = len(Kl)
        assert n_loc == L.mfc_kv_local_len(pos + 1, rank, WORLD, BLOCK)
        if n_loc:
            o, m, l = O.sdpa_partial(0, n_loc, q, np.stack(Kl), np.stack(Vl))
        else:
            o, m, l = np.zeros((H, D), np.float32), np.full(H, -np.inf, np.float32), np.zeros(H, np.float32)
        part = torch.tensor(np.concatenate([o.reshape(-1), m, l]))
        gathered = torch.empty(WORLD * part.numel())
        dist.all_gather_into_tensor(gathered, part)
        g = gathered.numpy().reshape(WORLD, -1)
        got = O.lse_merge_gate(g[:, :H * D].reshape(WORLD, H, D), g[:, H * D:H * D + H], g[:, H * D + H:], gate)
        ref = O.sdpa(pos + 1, q, gate, K[:pos + 1], V[:pos + 1])
        worst = max(worst, I.rel_err(got, ref))
    # every position has exactly one owner across the ranks
    owned = torch.zeros(ctx_len + n_steps)
    for p in range(ctx_len + n_steps):
        if L.mfc_kv_local_row(p, rank, WORLD, BLOCK) >= 0:
            owned[p] = 1
    dist.all_reduce(owned)
    assert bool((owned == 1).all())
    # GatedDeltaNet sequences: round-robin, disjoint, complete
    mine = torch.zeros(8)
    for s in range(8):
        if s % WORLD == rank:
            mine[s] = 1
    dist.all_reduce(mine)
    assert bool((mine == 1).all())
    w = torch.tensor([worst], dtype=torch.float64)
    dist.all_reduce(w, op=dist.ReduceOp.MAX)
    if rank == 0:
        with open(result_path, "w") as f:
            f.write(repr(float(w[0])))
    dist.destroy_process_group()


@pytest.mark.parametrize("ctx_len", [0, 100])
def test_kv_split_two_ranks_gloo(tmp_path, ctx_len):
    O.build()
    path = str(tmp_path / "worst.txt")
    mp.spawn(_worker, args=(_free_port(), ctx_len, 70, path), nprocs=WORLD, join=True)
    worst = float(open(path).read())
    assert worst <= 1e-5, worst


def _ragged_worker(rank, port, result_path):
    """Sharding by sequence (bench.py --workload ragged) on CPU ranks: each rank computes the layer-steps of its shard
    with the oracle, the padded outputs are all-gathered, and every sequence's output is found where the plan says."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=WORLD)
    import bench

    lens = [1 + (x % 97) for x in bench.ragged_lengths()]  # the benchmark's seeded lengths, scaled down for the CPU
    shards, load = bench.ragged_shards(lens, WORLD)
    n_max = max(len(s) for s in shards)
    mine = shards[rank]
    out = torch.zeros(n_max, G.q_dim)
    refs = {}
    for s in range(len(lens)):
        r = I.rng(7000 + s)  # per-sequence stream: every rank can form any sequence's reference
        K, V = I.normal(r, (lens[s], G.kv_dim)), I.normal(r, (lens[s], G.kv_dim))
        q, gate = I.normal(r, G.q_dim), I.normal(r, G.q_dim)
        o = O.sdpa(lens[s], q, gate, K, V)
        if s in mine:
            out[mine.index(s)] = torch.tensor(o)
        refs[s] = o
    gathered = torch.empty(WORLD * n_max, G.q_dim)
    dist.all_gather_into_tensor(gathered, out)
    ok = all(np.array_equal(gathered[rk * n_max + j].numpy(), refs[s]) for rk in range(WORLD) for j, s in enumerate(shards[rk]))
    flag = torch.tensor([1.0 if ok else 0.0])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        with open(result_path, "w") as f:
            f.write(repr((float(flag[0]), load)))
    dist.destroy_process_group()


def test_ragged_sequence_sharding_two_ranks_gloo(tmp_path):
    O.build()
    path = str(tmp_path / "ragged.txt")
    mp.spawn(_ragged_worker, args=(_free_port(), path), nprocs=WORLD, join=True)
    ok, load = eval(open(path).read())
    assert ok == 1.0


def test_ragged_shards_are_a_balanced_partition():
    import bench

    lens = bench.ragged_lengths()
    assert len(lens) == 64 and min(lens) >= 1024 and max(lens) <= 32768
    assert lens == bench.ragged_lengths()  # seeded
    for world in (1, 2, 4, 8):
        shards, load = bench.ragged_shards(lens, world)
        assert sorted(s for sh in shards for s in sh) == list(range(64))      # every sequence exactly once
        assert [sum(lens[s] for s in sh) for sh in shards] == load
        assert max(load) - min(load) <= max(lens)                             # greedy longest-first bound
        assert max(load) <= 1.05 * sum(lens) / world + 1                      # and close to even for these lengths
