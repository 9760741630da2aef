"""CPU test of the label-sharding host logic with two gloo ranks.

The per-shard compute is injected: here it is the CPU oracle (test infrastructure), so the test
checks the partitioning, the target filtering and the all-reduce plumbing of
ecml23_sparse_b200.sharded, not the CUDA kernels.
"""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ecml23_sparse_b200 import sharded, synth


def test_shard_range_covers_everything_once():
    for total, world in [(10, 3), (670_091, 8), (5, 8), (16, 4), (1, 1)]:
        seen = []
        for r in range(world):
            lo, hi = sharded.shard_range(total, world, r)
            assert 0 <= lo <= hi <= total
            seen.extend(range(lo, hi))
        assert seen == list(range(total))
    with pytest.raises(ValueError):
        sharded.shard_range(10, 2, 2)


def test_filter_targets_rebases_labels():
    row_ptr = torch.tensor([0, 3, 3, 5], dtype=torch.int32)
    labels = torch.tensor([1, 7, 9, 0, 8], dtype=torch.int32)
    ptr, lab = sharded.filter_targets(row_ptr, labels, 5, 10)
    assert ptr.tolist() == [0, 2, 2, 3]
    assert lab.tolist() == [2, 4, 3]
    ptr, lab = sharded.filter_targets(row_ptr, labels, 0, 5)
    assert ptr.tolist() == [0, 1, 1, 2] and lab.tolist() == [1, 0]


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, out_dir: str):
    import oracle  # test infrastructure: stands in for the CUDA ops on these CPU ranks

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        B, N, L, K = 6, 20, 101, 4
        x = synth.normal(3, 0, (B, N))
        idx = synth.indices_without_replacement(3, 1, L, K, N)
        W = synth.normal(3, 2, (L, K), std=0.5)
        g = synth.normal(3, 3, (B, L))
        lo, hi = sharded.shard_range(L, world, rank)
        idx_s, W_s = idx[lo:hi].numpy(), W[lo:hi].numpy()
        xT = x.t().contiguous()

        def forward_fn(xT_):
            return torch.from_numpy(oracle.forward_f32(xT_.numpy(), idx_s, W_s, transposed=True))

        def backward_fn(xT_, g_s):
            gx = oracle.grad_x_f32(idx_s, W_s, g_s.numpy(), N, transposed=True)
            gw = oracle.grad_w_f32(xT_.numpy(), idx_s, g_s.numpy(), transposed=True)
            return torch.from_numpy(gx), torch.from_numpy(gw), torch.from_numpy(g_s.numpy().sum(0))

        # no symmetric (peer-visible) memory on CPU ranks: all ranks agree to keep the all-reduce
        assert sharded.PeerSum.create(N * B, torch.device("cpu")) is None
        step = sharded.LabelShardedStep(forward_fn, backward_fn)
        assert step.world == world
        y, gx, gW, gb = step.step(xT, lambda y_: g[:, lo:hi].contiguous())
        np.savez(os.path.join(out_dir, f"rank{rank}.npz"), y=y.numpy(), gx=gx.numpy(), gW=gW.numpy(), lo=lo, hi=hi)
    finally:
        dist.destroy_process_group()


def test_two_rank_label_sharding_matches_unsharded(tmp_path):
    import oracle

    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    B, N, L, K = 6, 20, 101, 4
    x = synth.normal(3, 0, (B, N)).numpy()
    idx = synth.indices_without_replacement(3, 1, L, K, N).numpy()
    W = synth.normal(3, 2, (L, K), std=0.5).numpy()
    g = synth.normal(3, 3, (B, L)).numpy()
    y_full = oracle.forward_f64(x, idx, W)
    gx_full = oracle.grad_x_f64(idx, W, g, N, transposed=True)
    gW_full = oracle.grad_w_f64(x, idx, g)
    parts = [np.load(tmp_path / f"rank{r}.npz") for r in range(world)]
    y = np.concatenate([p["y"] for p in parts], axis=1)
    gW = np.concatenate([p["gW"] for p in parts], axis=0)
    np.testing.assert_allclose(y, y_full, rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(gW, gW_full, rtol=1e-5, atol=1e-5)
    for p in parts:  # every rank holds the full sum after the all-reduce
        np.testing.assert_allclose(p["gx"], gx_full, rtol=1e-5, atol=1e-5)
    assert int(parts[0]["hi"]) == int(parts[1]["lo"]) == 51
