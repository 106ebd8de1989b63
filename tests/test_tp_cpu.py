"""CPU tests of the tensor-parallel host logic with two `gloo` ranks: sharding the MLP weights the way the
reference's shapes do (mlp.cu:243-251) and summing the row-parallel partial outputs reproduces the unsharded
layer; the max-over-ranks reduction used for timing."""
import os
import socket
import sys

import numpy as np
import pytest

torch = pytest.importorskip("torch")
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close()
    return p


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, os.path.dirname(HERE)); sys.path.insert(0, HERE)
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import oracle_lib as o
    from cusync_b200 import tp
    grp = tp.TensorParallelGroup(backend="gloo")
    rng = np.random.default_rng(0)                       # same full tensors on every rank
    B, H, F = 8, 256, 512
    x = rng.standard_normal((B, H)).astype(np.float16)
    w1 = (rng.standard_normal((H, F)) * 0.05).astype(np.float16)
    w2 = (rng.standard_normal((F, H)) * 0.05).astype(np.float16)
    w1s, w2s, _ = tp.shard_mlp_weights(torch.from_numpy(w1), torch.from_numpy(w2), None, world, rank)
    assert w1s.shape == (H, F // world) and w2s.shape == (F // world, H)
    # this rank's partial output through the oracle chain (fp16 intermediate, fp32 accumulate)
    h = o.gemm_f16(x, w1s.numpy(), o.EPI_GELU_ERF)
    y_part = torch.from_numpy(o.gemm_f16(h, w2s.numpy()).astype(np.float32))
    grp.all_reduce_sum(y_part)
    worst = grp.max_over_ranks(float(rank + 1))
    grp.barrier()
    if rank == 0:
        full = o.gemm_f16(o.gemm_f16(x, w1, o.EPI_GELU_ERF), w2).astype(np.float32)
        np.save(os.path.join(out_dir, "err.npy"),
                np.array([np.abs(y_part.numpy() - full).max() / np.abs(full).max(), worst]))
    grp.close()


def test_row_parallel_sum_reproduces_the_unsharded_layer(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    err, worst = np.load(os.path.join(str(tmp_path), "err.npy"))
    assert err <= 1e-2          # partials are rounded to fp16 before the sum
    assert worst == float(world)


def test_shard_bounds():
    sys.path.insert(0, os.path.dirname(HERE))
    from cusync_b200 import tp
    assert tp.shard_bounds(6144 * 8, 8, 3) == (3 * 6144, 4 * 6144)
    assert [tp.shard_bounds(8, 4, r) for r in range(4)] == [(0, 2), (2, 4), (4, 6), (6, 8)]
    with pytest.raises(ValueError):
        tp.shard_bounds(10, 4, 0)
