"""World-size-2 check of the data-parallel host logic on CPU (gloo): shard the
batch over ranks, compute the layer's weight/bias gradients per shard with the
oracle, sum them through the bucket's all-reduce, and compare with the
gradient of the whole batch."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    for p in (ROOT, os.path.join(ROOT, "cnn-mellin_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    import dp
    from oracle.oracle import Oracle

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        oracle = Oracle("port")
        rng = np.random.default_rng(0)  # identical data on every rank; each takes its slice
        n, ci, co, ng, nf = 5, 3, 4, (9, 24), (3, 3)
        s, d, p, u = (1, 1), (1, 1), (0, 1), (1, 1)
        x = rng.standard_normal((n, ci) + ng)
        w = rng.standard_normal((co, ci) + nf)
        y = oracle.mcorrlcorr(x, w, None, s, d, p, u, (6, 1))
        go = rng.standard_normal(y.shape)
        lo, hi = dp.shard_range(n, world, rank)
        _, gw, gb = oracle.mcorrlcorr_backward(np.ascontiguousarray(x[lo:hi]), w, np.ascontiguousarray(go[lo:hi]), s, d, p, u)
        bucket = dp.GradBucket([gw.shape, gb.shape], device="cpu", dtype=torch.float64)
        bucket.pack([torch.from_numpy(gw), torch.from_numpy(gb)])
        bucket.all_reduce()
        _, gw_full, gb_full = oracle.mcorrlcorr_backward(x, w, go, s, d, p, u)
        got_w, got_b = (v.numpy() for v in bucket.views())
        ok = np.allclose(got_w, gw_full, rtol=1e-12, atol=1e-12) and np.allclose(got_b, gb_full, rtol=1e-12, atol=1e-12)
        with open(os.path.join(out_dir, "rank%d" % rank), "w") as fp:
            fp.write("ok" if ok else "mismatch")
    finally:
        dist.destroy_process_group()


def test_sharded_gradients_sum_to_the_full_batch(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert (tmp_path / ("rank%d" % r)).read_text() == "ok"


def test_shard_helpers():
    sys.path.insert(0, os.path.join(ROOT, "cnn-mellin_b200"))
    import dp

    for total in (0, 1, 7, 32, 33):
        for world in (1, 2, 3, 8):
            ranges = [dp.shard_range(total, world, r) for r in range(world)]
            assert ranges[0][0] == 0 and ranges[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
            sizes = [e - b for b, e in ranges]
            assert max(sizes) - min(sizes) <= 1
    lengths = [800, 200, 750, 300, 500, 500, 640, 220]
    shards = dp.balanced_shards(lengths, 4)
    assert sorted(i for sh in shards for i in sh) == list(range(8))
    loads = [sum(lengths[i] for i in sh) for sh in shards]
    assert max(loads) - min(loads) <= 200
    with pytest.raises(ValueError):
        dp.shard_range(4, 2, 2)


def _reducer_worker(rank, world, port, out_dir):
    for p in (ROOT, os.path.join(ROOT, "cnn-mellin_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    import dp

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)  # identical model and data on every rank; each takes its slice of the batch
        model = torch.nn.Sequential(torch.nn.Linear(6, 16), torch.nn.ReLU(), torch.nn.Linear(16, 16), torch.nn.ReLU(),
                                    torch.nn.Linear(16, 3)).double()
        x, t = torch.randn(8, 6, dtype=torch.float64), torch.randn(8, 3, dtype=torch.float64)
        full = [g.clone() for g in torch.autograd.grad(((model(x) - t) ** 2).mean(), list(model.parameters()))]
        # small buckets: the six parameters spread over several of them
        reducer = dp.BucketedReducer(model.parameters(), bucket_bytes=1024)
        lo, hi = dp.shard_range(8, world, rank)
        ok = len(reducer.buckets) >= 2
        for step in range(2):  # the second step checks that the buckets are re-armed and re-zeroed
            reducer.begin_step()
            ((model(x[lo:hi]) - t[lo:hi]) ** 2).mean().backward()
            reducer.finish_step()
            for p_, g in zip(model.parameters(), full):
                ok = ok and torch.allclose(p_.grad, g, rtol=1e-12, atol=1e-14)
                ok = ok and p_.grad.data_ptr() >= reducer.buckets[reducer._bucket_of[p_]].data_ptr()
        with open(os.path.join(out_dir, "rank%d" % rank), "w") as fp:
            fp.write("ok" if ok else "mismatch")
    finally:
        dist.destroy_process_group()


def test_bucketed_reducer_averages_gradients_during_backward(tmp_path):
    world = 2
    mp.spawn(_reducer_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert (tmp_path / ("rank%d" % r)).read_text() == "ok"


def test_snake_shards_are_equal_count_and_balanced():
    sys.path.insert(0, os.path.join(ROOT, "cnn-mellin_b200"))
    import dp

    rng = np.random.default_rng(3)
    for world in (1, 2, 4, 8):
        lengths = rng.integers(200, 801, size=32 * world).tolist()
        shards = dp.snake_shards(lengths, world)
        assert sorted(i for sh in shards for i in sh) == list(range(32 * world))
        assert all(len(sh) == 32 for sh in shards)
        loads = [sum(lengths[i] for i in sh) for sh in shards]
        assert max(loads) - min(loads) <= 600  # under one utterance, against ~1000 (one sigma) for a random deal
    with pytest.raises(ValueError):
        dp.snake_shards([1, 2, 3], 2)
