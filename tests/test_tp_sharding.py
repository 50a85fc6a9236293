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


def test_shard_arithmetic():
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
