"""Tensor-parallel plumbing for the MLP / attention shards: one process per GPU, `torch.distributed` for the
single exchange step of a layer -- the sum all-reduce of the row-parallel output (the reference only ever
times this collective on its own, src/ml-bench/transformer/allreduce_times.py:11-35).

Sharding follows the reference's shapes (mlp.cu:243-251): rank r of P holds the r-th column slice of W1 (and V)
and the r-th row slice of W2; X is replicated; Y = sum_r act(X W1_r) W2_r.
"""
import os


def shard_bounds(total, parts, rank):
    """[begin, end) of `rank`'s slice when `total` columns/rows are split into `parts` equal slices."""
    if total % parts:
        raise ValueError("%d is not divisible into %d shards" % (total, parts))
    step = total // parts
    return rank * step, (rank + 1) * step


def shard_mlp_weights(w1, w2, v, parts, rank):
    """Column-parallel W1 / V, row-parallel W2 (Megatron split, as in mlp.cu:243-251)."""
    b, e = shard_bounds(w1.shape[1], parts, rank)
    return w1[:, b:e].contiguous(), w2[b:e, :].contiguous(), (v[:, b:e].contiguous() if v is not None else None)


class TensorParallelGroup:
    """World of the layer's ranks.  backend "nccl" on GPUs (NVLink/NVSwitch), "gloo" for the CPU tests."""

    def __init__(self, backend=None, device=None):
        import torch.distributed as dist
        self.dist = dist
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.device = device
        if self.world > 1 and not dist.is_initialized():
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")   # keep NCCL's banner off stdout
            kwargs = {}
            if backend in (None, "nccl") and device is not None:
                kwargs["device_id"] = device
            dist.init_process_group(backend or "nccl", **kwargs)

    def all_reduce_sum(self, tensor):
        """In-place sum over ranks; enqueued on the current stream for CUDA tensors."""
        if self.world > 1:
            self.dist.all_reduce(tensor)
        return tensor

    def all_reduce_rows_overlapped(self, shard, comm_stream, chunks=4):
        """Sum-all-reduce of shard.y in row blocks, each enqueued behind the 128-row tiles it covers instead of
        behind the whole second GEMM (the shard was built with post_rows=True and run_cusync has just been called).
        The collectives go to `comm_stream`; the caller joins it.  Row blocks are whole 128-row tiles, so every
        element is summed exactly as by one all-reduce of the whole matrix."""
        import torch
        tiles = (shard.batch + 127) // 128
        per = (tiles + chunks - 1) // chunks
        for first in range(0, tiles, per):
            n = min(per, tiles - first)
            shard.wait_rows(first, n, comm_stream)
            if self.world > 1:
                with torch.cuda.stream(comm_stream):
                    self.dist.all_reduce(shard.y[first * 128:min(shard.batch, (first + n) * 128)])

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()

    def max_over_ranks(self, value):
        """Largest `value` over ranks (how a multi-GPU time is reported)."""
        if self.world == 1:
            return float(value)
        import torch
        t = torch.tensor([float(value)], dtype=torch.float64, device=self.device if self.device is not None else "cpu")
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def close(self):
        if self.world > 1 and self.dist.is_initialized():
            self.dist.destroy_process_group()
