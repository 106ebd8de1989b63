"""GPU tests of the all-reduce kernel that runs beside the producing GEMM (cusync_allreduce_*) and of the
tensor-parallel layer built on it.  One rank on one GPU here (the kernel's waits, counters and the layer wiring);
the multi-rank checks run tests/tp_worker.py under torch.distributed.run when the box has two GPUs or more."""
import os
import subprocess
import sys

import numpy as np
import pytest

from cusync_b200 import mlp as M
from cusync_b200 import tp
from cusync_b200 import _lib as L

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def test_one_rank_allreduce_leaves_the_matrix_as_it_is_and_counts_its_runs():
    dev = torch.device("cuda")
    g = tp.TensorParallelGroup("nccl", dev)
    ar = tp.RowAllReduce(g, 300, 1024, dev, num_ctas=4)
    src = torch.randn((300, 1024), device=dev).half()
    for run in range(1, 4):
        ar.y.copy_(src)
        ar.run(torch.cuda.current_stream())
        torch.cuda.synchronize()
        assert ar.status_code() == 0
        assert torch.equal(ar.y, src)
        flags = ar.flags.cpu().numpy()
        assert flags[0] == run * ar.num_ctas               # the final handshake: one count per block and run
        assert (flags[8:8 + 3] == run).all()               # three row tiles, each published once per run
    ar.destroy()


def test_one_rank_layer_with_the_allreduce_beside_the_gemms():
    dev = torch.device("cuda")
    g = tp.TensorParallelGroup("nccl", dev)
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    for batch in (600, 2048):
        x, w1, w2, v = M.make_inputs("gpt3", batch, dev, seed=12)
        ar = tp.RowAllReduce(g, batch, M.GPT3_HIDDEN, dev, num_ctas=8)
        s = M.MLPShard("gpt3", batch, x, w1, w2, v, policy="rowsync", post_rows=True, max_ctas=sms - 8, y=ar.y)
        ref = M.MLPShard("gpt3", batch, x, w1, w2, v, policy="rowsync")
        ref.run_stream_ordered(torch.cuda.current_stream()); torch.cuda.synchronize()
        ps, cs_, rs = torch.cuda.Stream(priority=-1), torch.cuda.Stream(), torch.cuda.Stream()
        for _ in range(3):
            s.y.fill_(float("nan")); torch.cuda.synchronize()
            s.run_cusync_allreduce(ar, ps, cs_, rs)
            cs_.synchronize()                               # the consumer stream carries the finished layer
            assert s.status_codes() == (0, 0)
            assert ar.status_code() == 0, (batch, ar.describe_status(), ar.flags[:16].tolist())
            assert torch.equal(s.y, ref.y)
        plain = M.MLPShard("gpt3", batch, x, w1, w2, v, policy="rowsync")
        with pytest.raises(L.CuSyncError):                  # needs post_rows
            plain.run_cusync_allreduce(ar, ps, cs_, rs)
        plain.destroy(); s.destroy(); ref.destroy(); ar.destroy()


def test_allreduce_gives_up_when_its_rows_never_come():
    dev = torch.device("cuda")
    g = tp.TensorParallelGroup("nccl", dev)
    ar = tp.RowAllReduce(g, 256, 512, dev, num_ctas=2, timeout_ns=int(20e6))
    ar.y.fill_(1.0)
    sems = torch.zeros(2, dtype=torch.int32, device=dev)     # nothing ever posts these
    ar.run(torch.cuda.current_stream(), sems.data_ptr(), 1)
    torch.cuda.synchronize()                                 # returns: every wait inside is bounded
    assert ar.status_code() == L.ERROR_TIMEOUT
    assert (ar.y == 1.0).all()
    ar.destroy()


def test_multi_rank_allreduce_and_layer():
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs two GPUs or more (run under a multi-GPU allocation)")
    world = 2 if n < 4 else 4
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "tp_worker.py")
    env = dict(os.environ, NCCL_DEBUG="WARN")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world),
                        "--master-addr", "127.0.0.1", "--master-port", "29731", worker, "1024"],
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600, env=env)
    print(r.stdout[-4000:])
    assert r.returncode == 0
    assert r.stdout.count("TP_WORKER_OK") == world
