"""Two GPU ranks: the peer-push all-gather and a row-sharded projection against the single-GPU result.
Skipped on boxes with one GPU.  No rank fails on purpose here; the give-up path of the wait is bounded in
the kernel and reported through the status word."""
import os
import socket

import numpy as np
import pytest
import torch

from oracle import ref

pytestmark = pytest.mark.gpu


def _port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank(rank, world, port, out_dir):
    import torch.distributed as dist
    from ferrum_b200 import surface as S, tp
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        d = S.Device(rank, use_torch_stream=False)
        rows, cols, m = 512, 2048, 1
        per = rows // world
        comm = S.Comm(d, rank, world, 1 << 20)
        packed = ref.random_matrix(ref.Q4_K, rows, cols, seed=5)
        w = S.Matrix.from_packed(d, per, cols, 1, ref.Q4_K, tp.shard_packed(packed, ref.Q4_K, rows, cols, rank, world))
        x = torch.from_numpy(np.random.default_rng(6).standard_normal((m, cols)).astype(np.float32)).cuda()
        torch.cuda.synchronize()
        shard_bytes = m * per * 4
        for step in range(3):  # the same flag words are reused with rising sequence numbers
            y = comm.view(4096 + rank * shard_bytes, m * per)
            S.project(d, w, x * float(step + 1), m, y)
            comm.all_gather(4096, shard_bytes)
            d.synchronize()
            got = tp.gathered_to_rows(comm.view(4096, world * m * per), m, rows, world).cpu().numpy()
            want = ref.matmul(ref.Q4_K, packed, rows, cols, (x * float(step + 1)).cpu().numpy(), m)
            assert ref.rel_err(got, want) <= 1e-3, (rank, step)
        # captured: projection + gather replayed twice
        y = comm.view(4096 + rank * shard_bytes, m * per)
        d.capture_begin()
        S.project(d, w, x, m, y)
        comm.all_gather(4096, shard_bytes)
        g = d.capture_end()
        for _ in range(2):
            g.launch()
            d.synchronize()
        got = tp.gathered_to_rows(comm.view(4096, world * m * per), m, rows, world).cpu().numpy()
        assert ref.rel_err(got, ref.matmul(ref.Q4_K, packed, rows, cols, x.cpu().numpy(), m)) <= 1e-3
        dist.barrier()
        open(os.path.join(out_dir, f"ok{rank}"), "w").write("ok")
        comm.close()
    finally:
        dist.destroy_process_group()


def test_two_ranks_gather_a_sharded_projection(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_rank, args=(2, _port(), str(tmp_path)), nprocs=2, join=True)
    assert os.path.exists(tmp_path / "ok0") and os.path.exists(tmp_path / "ok1")
