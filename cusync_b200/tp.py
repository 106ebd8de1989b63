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


class RowAllReduce:
    """The all-reduce kernel that runs beside the producing GEMM (cusync_allreduce_*): owns the output matrix
    `y` [rows, cols] fp16 and the flag words, in memory every rank's kernel can reach.  With more than one rank
    that is torch's symmetric memory (one process per GPU; peer mappings and, where the NVSwitch offers it, a
    multicast address, both set up by a rendezvous over the process group); with one rank plain device memory.
    torch only provides the memory; the reduction is this library's kernel."""

    def __init__(self, group, rows, cols, device, num_ctas=8, multicast=True, timeout_ns=0):
        import ctypes as C
        import torch
        from . import _lib as L
        self.rows, self.cols, self.world, self.rank = rows, cols, group.world, group.rank
        words = int(L.lib().cusync_allreduce_flag_words(rows, 128))
        self.uses_multicast = False
        if group.world > 1:
            import torch.distributed._symmetric_memory as symm_mem
            self.y = symm_mem.empty((rows, cols), dtype=torch.half, device=device)
            self.flags = symm_mem.empty((max(words, 64),), dtype=torch.int32, device=device)
            self.flags.zero_()
            hy = symm_mem.rendezvous(self.y, group.dist.group.WORLD)
            hf = symm_mem.rendezvous(self.flags, group.dist.group.WORLD)
            self._handles = (hy, hf)
            bufs, flags = list(hy.buffer_ptrs), list(hf.buffer_ptrs)
            mc_y = int(hy.multicast_ptr or 0) if multicast else 0     # 0 where the box offers no NVLS multicast
            mc_f = int(hf.multicast_ptr or 0) if mc_y else 0
            if not (mc_y and mc_f):
                mc_y = mc_f = 0
            self.uses_multicast = bool(mc_y)
            torch.cuda.synchronize(device)
            group.barrier()                 # every rank's flags are zero before any rank's kernel can signal
        else:
            self.y = torch.empty((rows, cols), dtype=torch.half, device=device)
            self.flags = torch.zeros((max(words, 64),), dtype=torch.int32, device=device)
            bufs, flags, mc_y, mc_f = [self.y.data_ptr()], [self.flags.data_ptr()], 0, 0
        self._bufs = (C.c_void_p * len(bufs))(*bufs)
        self._flags = (C.c_void_p * len(flags))(*flags)
        d = L.AllReduceDesc(group.rank, group.world, rows, cols, cols, 128, num_ctas, self._bufs, self._flags,
                            mc_y or None, mc_f or None, int(timeout_ns))
        self._plan = C.c_void_p()
        L.check(L.lib().cusync_allreduce_plan_create(C.byref(self._plan), C.byref(d)), "cusync_allreduce_plan_create")
        self.num_ctas = int(L.lib().cusync_allreduce_plan_num_ctas(self._plan))

    def run(self, stream, row_semaphores=None, value=0):
        """The all-reduce alone: the matrix is taken as complete when the kernel starts, unless semaphores are given."""
        from . import _lib as L
        from .api import _stream_ptr
        L.check(L.lib().cusync_allreduce_run(self._plan, row_semaphores, value, _stream_ptr(stream)), "cusync_allreduce_run")

    def status(self):
        import ctypes as C
        from . import _lib as L
        st = L.Status()
        L.lib().cusync_allreduce_read_status(self._plan, C.byref(st))
        return st

    def status_code(self):
        return self.status().code

    def describe_status(self):
        st = self.status()
        return "code %d where %d tile_x %d sem_index %d seen %d expected %d" % (
            st.code, st.where, st.tile_x, st.sem_index, st.seen, st.expected)

    def destroy(self):
        from . import _lib as L
        if self._plan:
            L.lib().cusync_allreduce_plan_destroy(self._plan)
            self._plan = None


class NativeComm:
    """The NCCL communicator of the C ABI (cusync_tp_comm_*): created from a unique id that rank 0 draws and the
    process group hands round; cusync_tp_layer_run then runs a layer and its ncclAllReduce without Python's help."""

    def __init__(self, group):
        import ctypes as C
        from . import _lib as L
        self.group = group
        uid = (C.c_char * 128)()
        if group.rank == 0 and group.world > 1:
            L.check(L.lib().cusync_tp_unique_id(uid), "cusync_tp_unique_id")
        if group.world > 1:
            box = [bytes(uid)]
            group.dist.broadcast_object_list(box, src=0)
            uid = (C.c_char * 128).from_buffer_copy(box[0])
        self._h = C.c_void_p()
        L.check(L.lib().cusync_tp_comm_create(C.byref(self._h), group.world, group.rank, uid), "cusync_tp_comm_create")

    def all_reduce(self, tensor, stream):
        from . import _lib as L
        from .api import _stream_ptr
        L.check(L.lib().cusync_tp_all_reduce(self._h, tensor.data_ptr(), tensor.numel(), _stream_ptr(stream)),
                "cusync_tp_all_reduce")

    def layer_run(self, shard, producer_stream, consumer_stream, reducer=None, reduce_stream=None):
        """One layer of `shard` with its all-reduce (cusync_tp_layer_run)."""
        from . import _lib as L
        from .api import _stream_ptr
        L.check(L.lib().cusync_tp_layer_run(shard._h, self._h, reducer._plan if reducer is not None else None,
                                            shard.y.data_ptr(), shard.y.numel(), _stream_ptr(producer_stream),
                                            _stream_ptr(consumer_stream), _stream_ptr(reduce_stream)), "cusync_tp_layer_run")

    def destroy(self):
        from . import _lib as L
        if self._h:
            L.lib().cusync_tp_comm_destroy(self._h)
            self._h = None


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

    def all_gather_rows(self, full, rows_per_rank):
        """Every rank holds rows [rank, rank + 1) * rows_per_rank of `full`; afterwards every rank holds all of it
        (in place, on the current stream): how a replicated input reaches the ranks when each of them fetched
        one share of it from the host."""
        if self.world > 1:
            mine = full[self.rank * rows_per_rank:(self.rank + 1) * rows_per_rank]
            self.dist.all_gather_into_tensor(full[:self.world * rows_per_rank], mine)
        return full

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
