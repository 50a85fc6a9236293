"""Row-sharded tensor parallelism: host logic on CPU ranks (gloo, world size 2), bit parity on the GPU."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ferrum_b200 import tp
from oracle import ref


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, fmt, rows, cols, m, out_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        packed = ref.random_matrix(fmt, rows, cols, seed=3)
        x = np.random.default_rng(4).standard_normal((m, cols)).astype(np.float32)
        shard = tp.shard_packed(packed, fmt, rows, cols, rank, world)
        first, per = tp.shard_range(rows, rank, world)
        # The CPU oracle stands in for the device kernel here: this test is about slicing and gathering.
        y_part = torch.from_numpy(ref.matmul(fmt, shard, per, cols, x, m))
        gathered = torch.empty(world * m * per, dtype=torch.float32)
        dist.all_gather_into_tensor(gathered, y_part.reshape(-1).contiguous())
        y = tp.gathered_to_rows(gathered, m, rows, world).numpy()
        want = ref.matmul(fmt, packed, rows, cols, x, m)
        assert np.array_equal(y.view(np.uint32), want.view(np.uint32)), "gathered shards differ from the whole matrix"
        if rank == 0:
            np.save(out_path, y)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("fmt", [ref.Q4_K, ref.Q6_K, ref.Q8_0])
def test_two_cpu_ranks_reassemble_the_projection(tmp_path, fmt):
    rows, cols, m = 48, 512, 3
    out = str(tmp_path / "y.npy")
    mp.spawn(_rank_main, args=(2, free_port(), fmt, rows, cols, m, out), nprocs=2, join=True)
    assert np.load(out).shape == (m, rows)


def _ep_rank_main(rank, world, port, out_path):
    """Expert parallelism on CPU ranks: replicated routing, each rank computes the expert-sorted rows of its own
    experts (the oracle stands in for the kernels), the runs are exchanged, every rank combines."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        experts, used, hidden, ef, m = 8, 2, 256, 256, 5
        gate_e = ref.random_matrix(ref.Q4_K, experts * ef, hidden, 1)
        down_e = ref.random_matrix(ref.Q6_K, experts * hidden, ef, 2)
        x = (np.random.default_rng(3).standard_normal((m, hidden)) * 0.3).astype(np.float32)
        logits = np.random.default_rng(4).standard_normal((m, experts)).astype(np.float32)
        ids, wts, gate = ref.moe_route(logits, x, x[0], experts, used, hidden, m, False, True, False)
        offsets, sorted_, position = ref.moe_map(ids, experts)
        routes = m * used
        first, count = tp.expert_range(experts, rank, world)
        lo, hi = int(offsets[first]), int(offsets[first + count])
        xg = x[np.asarray(sorted_) // used]  # expert-sorted activation rows
        sorted_ids = np.asarray(ids).reshape(-1)[np.asarray(sorted_)]
        my_gate = tp.shard_experts(gate_e, ref.Q4_K, ef, hidden, experts, rank, world)
        my_down = tp.shard_experts(down_e, ref.Q6_K, hidden, ef, experts, rank, world)
        rows = np.zeros((routes, hidden), dtype=np.float32)
        if hi > lo:
            local = (sorted_ids[lo:hi] - first).astype(np.uint32)
            h = ref.matmul_id(ref.Q4_K, my_gate, ef, hidden, xg[lo:hi], local, 1)
            rows[lo:hi] = ref.matmul_id(ref.Q6_K, my_down, hidden, ef, h, local, 1)
        # variable-length all-gather: every rank contributes its run of rows
        runs = [None] * world
        dist.all_gather_object(runs, (lo, hi, rows[lo:hi].copy()))
        full = np.zeros_like(rows)
        for a, b, part in runs:
            full[a:b] = part
        zero = np.zeros((m, hidden), dtype=np.float32)
        got = ref.moe_combine(full, wts, position, zero, gate, hidden, used, m, identity=False)
        # one rank with every expert, identity order
        h1 = ref.matmul_id(ref.Q4_K, gate_e, ef, hidden, x, ids, used)
        d1 = ref.matmul_id(ref.Q6_K, down_e, hidden, ef, h1, ids, 1)
        want = ref.moe_combine(d1, wts, ids, zero, gate, hidden, used, m, identity=True)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), "expert-parallel result differs from one rank"
        if rank == 0:
            np.save(out_path, got)
    finally:
        dist.destroy_process_group()


def _ep_all_to_all_main(rank, world, port, out_path):
    """The wide-input exchange on CPU ranks: a rank's expert rows go only to the ranks that own their tokens, the
    owners combine their tokens, the outputs are gathered.  The oracle stands in for the kernels; what is under
    test is who sends what to whom and that every owner ends up with all rows of its tokens."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        experts, used, hidden, m = 12, 2, 64, 11
        rng = np.random.default_rng(5)
        logits = rng.standard_normal((m, experts)).astype(np.float32)
        x = rng.standard_normal((m, hidden)).astype(np.float32)
        ids, wts, gate = ref.moe_route(logits, x, x[0], experts, used, hidden, m, False, True, False)
        offsets, sorted_, position = ref.moe_map(ids, experts)
        routes = m * used
        # stand-in for the expert projections: row p of the sorted set depends on its route and its expert only
        sorted_ids = np.asarray(ids).reshape(-1)[np.asarray(sorted_)]
        all_rows = (np.asarray(sorted_)[:, None] * 1000 + sorted_ids[:, None] * 7 + np.arange(hidden)[None, :]).astype(np.float32)
        first, count = tp.expert_range(experts, rank, world)
        lo, hi = int(offsets[first]), int(offsets[first + count])
        per, token0, mine = tp.token_owner_range(m, rank, world)
        assert per % 4 == 0 and per * world >= m
        # dispatch: only to the owner of the row's token
        outbox = [[] for _ in range(world)]
        for p in range(lo, hi):
            outbox[tp.token_owner(int(sorted_[p]) // used, per, world)].append((p, all_rows[p]))
        gathered = [None] * world
        dist.all_gather_object(gathered, outbox)  # gloo has no object all-to-all: gather the outboxes, take this rank's column
        have = np.full((routes, hidden), np.nan, dtype=np.float32)
        received = 0
        for sender in range(world):
            for p, row in gathered[sender][rank]:
                have[p] = row
                received += 1
        assert received == mine * used, "an owner receives exactly the rows of its tokens"
        zero = np.zeros((m, hidden), dtype=np.float32)
        part = np.zeros((per, hidden), dtype=np.float32)
        if mine:
            sl = slice(token0, token0 + mine)
            sub_pos = np.asarray(position).reshape(m, used)[sl].reshape(-1)
            assert np.isfinite(have[sub_pos]).all()
            # combine the owner's tokens: the oracle on the sub-range, positions unchanged (they index the whole set)
            full = np.where(np.isfinite(have), have, 0).astype(np.float32)
            part[:mine] = ref.moe_combine(full, np.asarray(wts).reshape(m, used)[sl].reshape(-1), sub_pos, zero[sl],
                                          np.asarray(gate)[sl], hidden, used, mine, identity=False)
        outs = [None] * world
        dist.all_gather_object(outs, part)
        got = np.concatenate(outs)[:m]
        want = ref.moe_combine(all_rows, wts, position, zero, gate, hidden, used, m, identity=False)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
        if rank == 0:
            np.save(out_path, got)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_cpu_ranks_exchange_rows_with_the_token_owners(tmp_path, world):
    out = str(tmp_path / "a2a.npy")
    mp.spawn(_ep_all_to_all_main, args=(world, free_port(), out), nprocs=world, join=True)
    assert np.load(out).shape == (11, 64)


def test_token_owner_split():
    assert tp.token_owner_range(1024, 3, 8) == (128, 384, 128)
    assert tp.token_owner_range(40, 1, 2) == (20, 20, 20)
    assert tp.token_owner_range(41, 7, 8) == (8, 56, 0)      # the last ranks may own nothing
    assert tp.token_owner_range(41, 5, 8) == (8, 40, 1)
    assert tp.token_owner(40, 8, 8) == 5 and tp.token_owner(1000, 8, 8) == 7


def test_two_cpu_ranks_split_the_experts(tmp_path):
    out = str(tmp_path / "moe.npy")
    mp.spawn(_ep_rank_main, args=(2, free_port(), out), nprocs=2, join=True)
    assert np.load(out).shape == (5, 256)


def test_shard_arithmetic():
    assert tp.expert_range(256, 5, 8) == (160, 32)
    e = ref.random_matrix(ref.Q6_K, 4 * 2, 256, seed=2)  # 4 experts x 2 rows
    assert np.array_equal(tp.shard_experts(e, ref.Q6_K, 2, 256, 4, 1, 2), e[2 * 2 * 210:])
    assert tp.shard_range(17408, 3, 8) == (6528, 2176)
    with pytest.raises(ValueError):
        tp.shard_range(10, 0, 4)
    with pytest.raises(ValueError):
        tp.shard_range(8, 2, 2)
    packed = ref.random_matrix(ref.Q4_K, 3 * 8, 256, seed=1)  # 3 experts x 8 rows
    s1 = tp.shard_packed(packed, ref.Q4_K, 8, 256, 1, 2, experts=3)
    full = packed.reshape(3, 8, 144)
    assert np.array_equal(s1.reshape(3, 4, 144), full[:, 4:8])
    g = np.arange(2 * 3 * 4, dtype=np.float32)
    rows = tp.gathered_to_rows(g, 3, 8, 2)
    assert rows.shape == (3, 8) and rows[1, 5] == g[1 * 12 + 1 * 4 + 1]


@pytest.mark.gpu
@pytest.mark.parametrize("fmt,m", [(ref.Q4_K, 1), (ref.Q4_K, 8), (ref.Q6_K, 1), (ref.Q6_K, 16)])
def test_row_shards_give_the_bits_of_the_whole_matrix(device, fmt, m):
    """Parity for the sharded path: gathered shard outputs == the single-GPU output, bit for bit."""
    from ferrum_b200 import surface as S
    rows, cols, world = 256, 2048, 4
    packed = ref.random_matrix(fmt, rows, cols, seed=9)
    x = torch.from_numpy(np.random.default_rng(10).standard_normal((m, cols)).astype(np.float32)).cuda()
    whole = torch.zeros(m * rows, dtype=torch.float32, device="cuda")
    S.project(device, S.Matrix.from_packed(device, rows, cols, 1, fmt, packed), x, m, whole)
    parts = []
    for r in range(world):
        _, per = tp.shard_range(rows, r, world)
        w = S.Matrix.from_packed(device, per, cols, 1, fmt, tp.shard_packed(packed, fmt, rows, cols, r, world))
        y = torch.zeros(m * per, dtype=torch.float32, device="cuda")
        S.project(device, w, x, m, y)
        parts.append(y)
    device.synchronize()
    got = tp.gathered_to_rows(torch.cat(parts), m, rows, world).cpu().numpy()
    assert np.array_equal(got.view(np.uint32), whole.cpu().numpy().reshape(m, rows).view(np.uint32))
