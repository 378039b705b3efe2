"""Host-side logic of the N-sharded path with world_size 2 over gloo on CPU: the shard
bounds, the all_gather layout ([R, M, N/R] -> [M, N]) and expert-parallel ownership.  The
local matmul is stood in by the CPU checker (the CUDA kernels need a GPU)."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import oracle as O
    from mlx_b200.distributed import all_gather_columns, shard_bounds, shard_rows

    rng = np.random.default_rng(0)
    N, K, M, g, bits = 64, 128, 3, 32, 4
    w = (0.02 * rng.standard_normal((N, K))).astype(np.float32)
    x = rng.standard_normal((M, K)).astype(np.float32)
    wq, s, b = O.quantize(w, g, bits, "f32")
    full = O.qmm(x, wq, s, b, True, g, bits, "f32")
    lo, hi = shard_bounds(N, rank, world)
    # a shard of the packed rows is a plain slice: no repacking
    wq_r = shard_rows(torch.from_numpy(wq.view(np.int32)), rank, world).numpy().view(np.uint32)
    assert np.array_equal(wq_r, wq[lo:hi])
    y_r = O.qmm(x, wq_r, s[lo:hi], b[lo:hi], True, g, bits, "f32")
    y = all_gather_columns(torch.from_numpy(y_r), None, world).numpy()
    ok = bool(np.array_equal(y, full))
    # batched leading dims
    y3 = all_gather_columns(torch.from_numpy(np.stack([y_r, 2 * y_r])), None, world).numpy()
    ok = ok and bool(np.array_equal(y3[1], 2 * full))
    # K-sharded layer: column slices of the packed words / scale groups, partial products, all_sum
    from mlx_b200.distributed import QuantizedShardedToAllLinear
    layer = QuantizedShardedToAllLinear(torch.from_numpy(wq.view(np.int32)), torch.from_numpy(s), torch.from_numpy(b), g, bits,
                                        rank=rank, world=world)
    klo, khi = rank * K // world, (rank + 1) * K // world
    assert layer.k_local == K // world and tuple(layer.weight.shape) == (N, (K // world) * bits // 32)
    assert np.array_equal(layer.weight.numpy().view(np.uint32), wq[:, klo * bits // 32:khi * bits // 32])
    xs = layer.x_slice(torch.from_numpy(x)).numpy()
    assert np.array_equal(xs, x[:, klo:khi])
    part = O.qmm(xs, layer.weight.numpy().view(np.uint32), layer.scales.numpy(), layer.biases.numpy(), True, g, bits, "f32")
    tot = torch.from_numpy(part.copy())
    dist.all_reduce(tot)
    ok = ok and bool(np.allclose(tot.numpy(), full, rtol=1e-5, atol=1e-5))
    ret[rank] = ok
    dist.destroy_process_group()


def test_n_sharded_all_gather_gloo_world2():
    world = 2
    port = 29500 + (os.getpid() % 2000)
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
        assert all(ret.get(r) for r in range(world))


def test_shard_bounds_errors():
    from mlx_b200.distributed import expert_bounds, shard_bounds
    assert shard_bounds(14336, 3, 8) == (5376, 7168)
    assert expert_bounds(8, 7, 8) == (7, 8)
    with pytest.raises(ValueError):
        shard_bounds(10, 0, 4)
    with pytest.raises(ValueError):
        shard_bounds(8, 4, 4)
