"""Host logic of the data-parallel path on CPU: two gloo ranks exchange gradients through GradReducer."""
import os
import socket

import numpy as np
import pytest

from helium_b200.grad_sync import GradReducer, bucket_by_bytes, shard_rows


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, mean, out_dir):
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        red = GradReducer(mean=mean)
        assert red.enabled and red.world == world
        # what a rank's backward pass would produce for its token shard: dW = X_shard^T dZ_shard, db = colsum
        g = np.random.Generator(np.random.Philox(7))
        x = g.standard_normal((64, 8)); dz = g.standard_normal((64, 12))
        rows = shard_rows(64, world, rank)
        xs, dzs = x[rows.start:rows.stop], dz[rows.start:rows.stop]
        flat = torch.zeros(8 * 12 + 12, dtype=torch.float64)
        dw = flat[:96].view(8, 12); db = flat[96:]
        dw.copy_(torch.from_numpy(xs.T @ dzs)); db.copy_(torch.from_numpy(dzs.sum(0)))
        red.reduce_bucket([dw])
        red.reduce_bucket([db])
        red.finish()
        red.reduce_bucket([])     # an empty bucket is a no-op
        red.finish()
        np.save(os.path.join(out_dir, f"r{rank}.npy"), flat.numpy())
        assert red.collectives == 2 and red.bytes_reduced == flat.numel() * 8
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mean", [True, False])
def test_two_ranks_reduce_sharded_gradients(tmp_path, mean):
    import torch.multiprocessing as mp
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), mean, str(tmp_path)), nprocs=world, join=True)
    g = np.random.Generator(np.random.Philox(7))
    x = g.standard_normal((64, 8)); dz = g.standard_normal((64, 12))
    full = np.concatenate([(x.T @ dz).reshape(-1), dz.sum(0)])
    want = full / world if mean else full
    for r in range(world):
        got = np.load(tmp_path / f"r{r}.npy")
        assert np.allclose(got, want, rtol=1e-12, atol=1e-12)


def test_single_process_is_a_no_op():
    import torch
    red = GradReducer()
    assert not red.enabled and red.world == 1
    t = torch.ones(4)
    red.reduce_bucket([t]); red.finish()
    assert torch.equal(t, torch.ones(4)) and red.collectives == 0


def test_shard_rows_covers_everything_once():
    for total, world in [(8192, 8), (10, 4), (3, 8), (0, 2), (7, 1)]:
        seen = []
        for r in range(world):
            rows = shard_rows(total, world, r)
            seen.extend(rows)
            assert len(rows) in (total // world, total // world + 1)
        assert seen == list(range(total))


def test_bucket_by_bytes():
    assert bucket_by_bytes([10, 10, 10, 10], 20) == [[0, 1], [2, 3]]
    assert bucket_by_bytes([50, 1, 1], 20) == [[0], [1, 2]]
    assert bucket_by_bytes([], 20) == []
    assert bucket_by_bytes([1, 1, 1], 100) == [[0, 1, 2]]
