"""Worker of the multi-GPU tests: one process per GPU under torch.distributed.run (NCCL).  Not a test module.

Checks, on every rank: (1) the all-reduce kernel alone (multicast form where the box offers it, and the plain
peer load/store form) against the fp32 sum of the ranks' matrices; (2) the tensor-parallel GPT-3 MLP shard with
the all-reduce overlapped (cusync_mlp_run_cusync_allreduce) against the same shard followed by NCCL's all-reduce.
Prints "TP_WORKER_OK <rank>" on success.
"""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

from cusync_b200 import mlp as M  # noqa: E402
from cusync_b200 import tp  # noqa: E402


def main():
    batch = int(sys.argv[1]) if len(sys.argv) > 1 else 1024
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    g = tp.TensorParallelGroup("nccl", dev)
    rows, cols = 300, 1024
    for multicast in (True, False):
        ar = tp.RowAllReduce(g, rows, cols, dev, num_ctas=4, multicast=multicast)
        if multicast and g.rank == 0:
            print("multicast addresses in use: %s" % ar.uses_multicast, flush=True)
        gen = torch.Generator(device=dev).manual_seed(100 + g.rank)
        for run in range(3):
            mine = torch.randn((rows, cols), generator=gen, device=dev).half()
            ar.y.copy_(mine)
            parts = [torch.empty_like(mine) for _ in range(g.world)]
            g.dist.all_gather(parts, mine)
            expect = sum(p.float() for p in parts).half()
            torch.cuda.synchronize(); g.barrier()
            ar.run(torch.cuda.current_stream())
            torch.cuda.synchronize(); g.barrier()
            assert ar.status_code() == 0
            # fp32 accumulation of at most 8 halves, one rounding: at most one half ulp from the rank-order sum
            assert torch.allclose(ar.y.float(), expect.float(), rtol=2e-3, atol=1e-3), (multicast, run)
        ar.destroy()

    # the sharded layer: every rank its own weights (seeded by rank), X replicated
    x, _, _, _ = M.make_inputs("gpt3", batch, dev, seed=0)
    _, w1, w2, _ = M.make_inputs("gpt3", batch, dev, seed=10 + g.rank)
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    ar = tp.RowAllReduce(g, batch, M.GPT3_HIDDEN, dev, num_ctas=8)
    over = M.MLPShard("gpt3", batch, x, w1, w2, None, policy="rowsync", post_rows=True, max_ctas=sms - ar.num_ctas, y=ar.y)
    ref = M.MLPShard("gpt3", batch, x, w1, w2, None, policy="rowsync")
    ps, cs, rs = torch.cuda.Stream(priority=-1), torch.cuda.Stream(), torch.cuda.Stream()
    ref.run_stream_ordered(cs)
    with torch.cuda.stream(cs):
        g.all_reduce_sum(ref.y)
    torch.cuda.synchronize(); g.barrier()
    for run in range(3):
        over.y.fill_(float("nan")); torch.cuda.synchronize(); g.barrier()
        over.run_cusync_allreduce(ar, ps, cs, rs)
        cs.synchronize()
        torch.cuda.synchronize(); g.barrier()
        assert over.status_codes() == (0, 0) and ar.status_code() == 0
        assert not torch.isnan(over.y.float()).any()
        scale = ref.y.float().abs().max().item()
        err = (over.y.float() - ref.y.float()).abs().max().item()
        assert err <= 4e-3 * scale, (run, err, scale)          # two fp16 roundings of sums ordered differently
    # the same two forms through the C ABI's own driver and communicator (cusync_tp_*): NCCL is called from C
    comm = tp.NativeComm(g)
    plain = M.MLPShard("gpt3", batch, x, w1, w2, None, policy="rowsync")
    for run in range(2):
        plain.y.fill_(float("nan")); over.y.fill_(float("nan")); torch.cuda.synchronize(); g.barrier()
        comm.layer_run(plain, ps, cs)
        comm.layer_run(over, ps, cs, reducer=ar, reduce_stream=rs)
        torch.cuda.synchronize(); g.barrier()
        if plain.tail_splits[:2] == ref.tail_splits[2:]:
            assert torch.equal(plain.y, ref.y)                   # same kernels, same NCCL all-reduce
        else:                                                    # K slices in the last partial round of one arm only
            perr = (plain.y.float() - ref.y.float()).abs().max().item()
            assert perr <= 4e-3 * ref.y.float().abs().max().item()
        err = (over.y.float() - ref.y.float()).abs().max().item()
        assert err <= 4e-3 * ref.y.float().abs().max().item()
    t = torch.full((1000,), float(g.rank + 1), device=dev, dtype=torch.half)
    comm.all_reduce(t, torch.cuda.current_stream()); torch.cuda.synchronize()
    assert (t == sum(range(1, g.world + 1))).all()
    plain.destroy(); comm.destroy()
    over.destroy(); ref.destroy(); ar.destroy()
    print("TP_WORKER_OK %d" % g.rank, flush=True)
    g.close()


if __name__ == "__main__":
    main()
