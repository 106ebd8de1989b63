#!/usr/bin/env python
"""Benchmark of the hot path: one GPT-3 175B MLP layer, one 8-way
tensor-parallel shard, as a chain of two tile-synchronised GEMMs.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch B] [--policy rowsync|tilesync]
    python bench.py --impl reference ...          # the CPU host-reference path, timed on the host cores

A step is one MLP layer over one batch of synthetic input (X ~ N(0,1),
weights ~ N(0,0.02), seeded): producer GEMM (+GELU) on one stream, wait kernel
and consumer GEMM on another, semaphores between them; with N > 1 GPUs an NCCL
all-reduce of the [B, 12288] output follows on the consumer stream.  One JSON
line is printed by rank 0.  Time-like metric: microseconds per layer.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

REDUCE_CHUNKS = 4
METRIC = "gpt3_mlp_layer_latency"
UNIT = "us"
SWEEP_BATCHES = [1, 64, 256, 512, 1024, 2048]


_RESULT_FD = None


def claim_stdout():
    """Keeps the process's stdout for the result line alone: libraries that write to file descriptor 1 (NCCL's
    version banner) go to stderr from here on."""
    global _RESULT_FD
    sys.stdout.flush()
    _RESULT_FD = os.dup(1)
    os.dup2(2, 1)


def emit(line):
    data = (json.dumps(line) + "\n").encode()
    if _RESULT_FD is None:
        sys.stdout.write(data.decode()); sys.stdout.flush()
    else:
        os.write(_RESULT_FD, data)


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "tflops_burst": p["bf16_tflops"],
                "tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "tflops_burst": 1590.0, "tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 7:
                continue
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
            except ValueError:
                continue
            for name, val in zip(names, r[3:7]):
                if val.lower().startswith("active") and not val.lower().startswith("not"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def cpu_reference_us(batch, sample_rows, hidden, ffn):
    """The CPU host-reference path (oracle restatement of ref_cpumatmul + GELU) on `sample_rows` rows of the
    layer, all host threads; returns (microseconds scaled to `batch` rows, threads, seconds spent)."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import numpy as np
    import oracle_lib as o
    rng = np.random.default_rng(0)
    x = rng.standard_normal((sample_rows, hidden), dtype=np.float32).astype(np.float16)
    w1 = (rng.standard_normal((hidden, ffn), dtype=np.float32) * 0.02).astype(np.float16)
    w2 = (rng.standard_normal((ffn, hidden), dtype=np.float32) * 0.02).astype(np.float16)
    o.gemm_f16(x[:16], w1, o.EPI_GELU_ERF)   # warm the library and the thread pool
    t0 = time.perf_counter()
    h = o.gemm_f16(x, w1, o.EPI_GELU_ERF)
    o.gemm_f16(h, w2)
    dt = time.perf_counter() - t0
    return dt * 1e6 * batch / sample_rows, o.num_threads(), dt


def run_reference(args, rank, world):
    """--impl reference: the reference's CPU check path for this layer, on the host cores.  Its CUTLASS GPU
    kernels cannot be built (un-vendored, un-pinned CUTLASS submodule), so the CPU path is the oracle's
    restatement of ref_cpumatmul (kind "port")."""
    if rank != 0:
        return
    from cusync_b200 import mlp as M
    hidden, ffn = M.GPT3_HIDDEN, M.GPT3_FFN
    sample = min(args.batch, 1024)
    times = []
    for i in range(args.warmup + args.steps):
        us, threads, _ = cpu_reference_us(args.batch, sample, hidden, ffn)
        if i >= args.warmup:
            times.append(us)
    val = statistics.mean(times)
    line = {"impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": val / 1000.0, "higher_is_better": False,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": workload_config(args, None),
            "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "kind": "port",
                             "sample": "%d of %d rows through both GEMMs, scaled to the full batch" % (sample, args.batch)},
            "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    emit(line)


def workload_config(args, shard):
    cfg = {"workload": "GPT-3 175B MLP, one 8-way tensor-parallel shard: X[%d,12288] * W1[12288,6144] -> GELU -> "
                       "* W2[6144,12288]" % args.batch,
           "batch": args.batch, "policy": args.policy,
           "l2": "inputs larger than L2 (302 MB of weights per step vs 126 MB L2); no explicit flush",
           "all_reduce": ("NCCL sum of Y[B,12288] fp16 across ranks" + (
               "; overlapped arm: %d row blocks, each behind the RowSync semaphores of its 128-row tiles of the "
               "second GEMM (%d of 148 SMs to the GEMMs)" % (args.reduce_chunks, args.gemm_ctas) if args.gpus > 1 and args.batch >= 512 and args.reduce == "overlapped" else ""))
                         if args.gpus > 1 else "none (1 GPU)"}
    if shard is not None:
        cfg.update({"tile_m": 128, "tile_n1": shard.tile_n1, "tile_n2": shard.tile_n2,
                    "ctas1": shard.ctas1, "ctas2": shard.ctas2, "split_k1": shard.split_k1, "split_k2": shard.split_k2,
                    "kernel": "CTA pairs (tcgen05 cta_group::2), 256x256 tile per pair" if args.batch > 256
                              else "one CTA per 128x256 tile"})
    return cfg


def time_steps(step_fn, start_stream, end_stream, steps, warmup, barrier):
    """Runs warmup + steps; returns (total ms over the K timed steps, per-step ms list)."""
    import torch
    for _ in range(warmup):
        step_fn()
    torch.cuda.synchronize()
    barrier()
    torch.cuda.synchronize()
    begins = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    for i in range(steps):
        # steps are serialised (a step may not overwrite H while the previous consumer reads it), so the
        # begin mark goes after the previous step's last kernel
        if start_stream is not end_stream:
            start_stream.wait_stream(end_stream)
        begins[i].record(start_stream)
        step_fn()
        ends[i].record(end_stream)
    torch.cuda.synchronize()
    barrier()
    total = begins[0].elapsed_time(ends[-1])
    per = [b.elapsed_time(e) for b, e in zip(begins, ends)]
    return total, per


def _watchdog(seconds):
    """Ends the process if the run is still going after `seconds`: a stream that waits for a value nobody writes
    (a chain that gave up on a bounded wait upstream) must not keep the device busy."""
    import threading

    def bail():
        sys.stderr.write("bench.py: no result after %d s, giving up\n" % seconds)
        sys.stderr.flush()
        os._exit(3)
    t = threading.Timer(seconds, bail)
    t.daemon = True
    t.start()


def main():
    _watchdog(1500)
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=2048)
    ap.add_argument("--policy", default="rowsync", choices=["rowsync", "tilesync"])
    ap.add_argument("--impl", default="cusync", choices=["cusync", "reference"])
    ap.add_argument("--reduce", choices=("overlapped", "after"), default="after",
                    help="multi-GPU: all-reduce Y after the second GEMM (default, the faster one here: NCCL needs "
                         "more SMs for full NVLink bandwidth than the GEMMs can spare), or in row blocks behind "
                         "the second GEMM's tiles")
    ap.add_argument("--reduce-chunks", type=int, default=REDUCE_CHUNKS, help="row blocks of the overlapped all-reduce")
    ap.add_argument("--gemm-ctas", type=int, default=128, help="blocks the GEMMs use when the all-reduce is overlapped")
    ap.add_argument("--no-sweep", action="store_true", help="skip the per-batch table")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    args = ap.parse_args()
    claim_stdout()
    args.warmup = max(args.warmup, 3) if args.impl == "cusync" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch
    from cusync_b200 import mlp as M
    from cusync_b200 import tp
    from cusync_b200 import _lib as L
    L.lib()   # fail loudly here if the CUDA library is not built
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the hot path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    group = tp.TensorParallelGroup("nccl", dev)

    def barrier():
        group.barrier()

    peaks = load_peaks()
    ps = torch.cuda.Stream(priority=-1)   # producer: high priority, launched first
    cs = torch.cuda.Stream(priority=0)

    comm = torch.cuda.Stream(priority=0)  # multi-GPU: the row-block all-reduces of the overlapped arm
    # Multi-GPU: the second GEMM also posts its output by 128-row tile, so that the all-reduce runs block by
    # block behind it; 20 SMs are left to the collective's kernels (128 blocks: 192 and 384 pair tiles are
    # whole rounds of 64 pairs, so the GEMMs lose nothing at B = 2048).
    overlap_reduce = world > 1 and args.batch >= 512 and args.reduce == "overlapped"

    def build(batch, policy):
        x, w1, w2, v = M.make_inputs("gpt3", batch, dev, seed=rank)
        if overlap_reduce:
            return M.MLPShard("gpt3", batch, x, w1, w2, v, policy=policy, post_rows=True, max_ctas=args.gemm_ctas)
        return M.MLPShard("gpt3", batch, x, w1, w2, v, policy=policy)

    shard = build(args.batch, args.policy)

    def cusync_step():
        # (the driver orders a run after the previous one: a step may not overwrite H while it is still read)
        shard.run_cusync(ps, cs)
        if overlap_reduce:
            group.all_reduce_rows_overlapped(shard, comm, args.reduce_chunks)
            cs.wait_stream(comm)
        elif world > 1:
            with torch.cuda.stream(cs):
                group.all_reduce_sum(shard.y)

    def ordered_step():
        shard.run_stream_ordered(cs)
        if world > 1:
            with torch.cuda.stream(cs):
                group.all_reduce_sum(shard.y)

    def reduce_max(v):
        return group.max_over_ranks(v)

    def interleaved(step_a, a_streams, step_b, b_streams, n, warm):
        """Alternates the two arms step by step, so clock and power drift hits both alike.
        Returns the per-step millisecond lists of A and B."""
        for _ in range(warm):
            step_a(); step_b()
        torch.cuda.synchronize()
        ev = []
        for _ in range(n):
            pair = []
            for fn, (s0, s1) in ((step_a, a_streams), (step_b, b_streams)):
                s0.wait_stream(cs); s0.wait_stream(ps)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(s0); fn(); e1.record(s1)
                pair.append((e0, e1))
            ev.append(pair)
        torch.cuda.synchronize()
        return [p[0][0].elapsed_time(p[0][1]) for p in ev], [p[1][0].elapsed_time(p[1][1]) for p in ev]

    if overlap_reduce:
        # the block-wise reduction must give what one all-reduce of the whole output gives
        cusync_step(); torch.cuda.synchronize()
        y_blocks = shard.y.clone()
        ordered_step(); torch.cuda.synchronize()
        if not torch.equal(y_blocks, shard.y):
            raise SystemExit("row-block all-reduce differs from the whole-matrix all-reduce")

    # ---- headline: overlapped chain ------------------------------------------------------------
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    total_ms, per_ms = time_steps(cusync_step, ps, cs, args.steps, args.warmup, barrier)
    total_ms = reduce_max(total_ms)
    ms_per_step = total_ms / args.steps
    codes = shard.status_codes()
    if codes != (0, 0):
        raise SystemExit("a bounded wait expired during the timed region: %r" % (codes,))

    # ---- same kernels serialised by stream order --------------------------------------------
    ord_total, ord_per = time_steps(ordered_step, cs, cs, args.steps, args.warmup, barrier)
    ord_ms = reduce_max(ord_total) / args.steps
    # ... and both arms interleaved step by step (the fair comparison under clock drift)
    il_c, il_o = interleaved(cusync_step, (ps, cs), ordered_step, (cs, cs), args.steps, 3)
    il_c_us, il_o_us = statistics.median(il_c) * 1000.0, statistics.median(il_o) * 1000.0

    # ---- per-kernel durations (stream-ordered, events on the launching stream) ----------------
    flops2 = 2.0 * args.batch * M.GPT3_FFN * M.GPT3_HIDDEN
    evs = []
    for i in range(args.warmup + args.steps):     # back to back, like the timed region: no host sync in between
        e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        e0.record(cs)
        shard.run_single(1, cs)
        e1.record(cs)
        shard.run_single(2, cs)
        e2.record(cs)
        if i >= args.warmup:
            evs.append((e0, e1, e2))
    torch.cuda.synchronize()
    g1 = [a.elapsed_time(b) for a, b, _ in evs]
    g2 = [b.elapsed_time(c) for _, b, c in evs]
    t1_ms, t2_bracketed_ms = statistics.mean(g1), statistics.mean(g2)
    # The consumer GEMM alone, `steps` launches back to back between ONE pair of events: the average launch
    # duration without an event record (a submission and a pipeline drain of its own) around every launch.
    for _ in range(args.warmup):
        shard.run_single(2, cs)
    l0, l1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    l0.record(cs)
    for _ in range(args.steps):
        shard.run_single(2, cs)
    l1.record(cs)
    torch.cuda.synchronize()
    t2_ms = l0.elapsed_time(l1) / args.steps
    # dram__bytes_read.sum + dram__bytes_write.sum of one launch of the consumer GEMM, from the ncu captures
    # summarised in profiles/cusync_gemm_pair_kernel_gpt3_mlp.md (bytes; None where no capture exists)
    traffic = {512: 222.6e6, 2048: 688.9e6}.get(args.batch)
    tensor_bound = args.batch >= 256
    kernel_name = ("cusync_gemm_pair_kernel (GEMM2, the consumer)" if args.batch > 256
                   else "cusync_gemm_kernel<%d,0> (GEMM2, the consumer)" % shard.tile_n2)
    if tensor_bound:
        achieved = flops2 / (t2_ms * 1e-3) / 1e12
        peak = peaks["tflops_sustained"]
        roofline = {"bound": "tensor", "kernel": kernel_name,
                    "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                    "peak_kind": "%s sustained bf16/fp16 cuBLAS" % peaks["source"],
                    "frac_of_burst_peak": achieved / peaks["tflops_burst"], "traffic": traffic,
                    "launch_ms": t2_ms, "launch_ms_event_bracketed": t2_bracketed_ms, "gemm1_ms": t1_ms,
                    "how": "launch_ms = consumer GEMM alone, steps launches back to back between one pair of events",
                    "gemm1_tflops": flops2 / (t1_ms * 1e-3) / 1e12}
    else:
        bytes2 = 2.0 * (M.GPT3_FFN * M.GPT3_HIDDEN + args.batch * (M.GPT3_FFN + M.GPT3_HIDDEN))
        achieved = bytes2 / (t2_ms * 1e-3) / 1e9
        roofline = {"bound": "hbm", "kernel": kernel_name,
                    "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                    "peak_kind": "%s copy bandwidth" % peaks["source"], "traffic": traffic, "launch_ms": t2_ms,
                    "launch_ms_event_bracketed": t2_bracketed_ms, "gemm1_ms": t1_ms}

    # ---- end to end through the C ABI with host buffers ---------------------------------------
    xh = torch.empty((args.batch, M.GPT3_HIDDEN), dtype=torch.half).pin_memory()
    xh.copy_(shard.x.cpu())
    yh = torch.empty((args.batch, M.GPT3_HIDDEN), dtype=torch.half).pin_memory()

    # One GPU: the result goes back to the host in row blocks, each behind the RowSync semaphores of its 128-row
    # tiles of the second GEMM (post_rows), so the device-to-host copy overlaps that GEMM.  Each GEMM gets half of
    # the SMs here: a persistent kernel that holds every SM while it waits for rows of X keeps the second GEMM
    # from becoming resident, and with it the first rows of Y from leaving while the last rows of X arrive.  The
    # step is bound by the PCIe link, not by the GEMMs, so halving their rate costs nothing.
    e2e_shard = shard
    d2h_blocks = 4
    if world == 1 and args.batch >= 512:
        d2h_blocks = max(4, min(8, args.batch // 256))
        e2e_ctas = torch.cuda.get_device_properties(dev).multi_processor_count // 4 * 2
        e2e_shard = M.MLPShard("gpt3", args.batch, shard.x, shard.w1, shard.w2, None, policy=args.policy, post_rows=True,
                               x_rows=True, max_ctas=e2e_ctas, group_rows2=2)
    d2h, h2d, post = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    landed = [torch.cuda.Event() for _ in range(d2h_blocks)]

    def e2e_step():
        ps.wait_stream(cs)
        tiles = (args.batch + 127) // 128
        per = (tiles + d2h_blocks - 1) // d2h_blocks
        if e2e_shard is not shard:
            # X comes in row blocks on its own stream, each followed by the post of its RowSync semaphores; the
            # first GEMM is launched right away and takes the rows as they land (x_rows)
            h2d.wait_stream(ps)
            post.wait_stream(ps)
            for first in range(0, tiles, per):
                n = min(per, tiles - first)
                r0, r1 = first * 128, min(args.batch, (first + n) * 128)
                with torch.cuda.stream(h2d):
                    e2e_shard.x[r0:r1].copy_(xh[r0:r1], non_blocking=True)
                # the post goes to a stream of its own behind an event, so that the copies stay back to back
                ev = landed[first // per]
                ev.record(h2d)
                post.wait_event(ev)
                e2e_shard.post_x_rows(first, n, post)
        else:
            with torch.cuda.stream(ps):
                e2e_shard.x.copy_(xh, non_blocking=True)
        e2e_shard.run_cusync(ps, cs)
        if e2e_shard is not shard:
            for first in range(0, tiles, per):
                n = min(per, tiles - first)
                e2e_shard.wait_rows(first, n, d2h)
                r0, r1 = first * 128, min(args.batch, (first + n) * 128)
                with torch.cuda.stream(d2h):
                    yh[r0:r1].copy_(e2e_shard.y[r0:r1], non_blocking=True)
            cs.wait_stream(d2h)
        else:
            with torch.cuda.stream(cs):
                group.all_reduce_sum(e2e_shard.y)
                yh.copy_(e2e_shard.y, non_blocking=True)

    e2e_total, _ = time_steps(e2e_step, ps, cs, args.steps, args.warmup, barrier)
    e2e_us = reduce_max(e2e_total) / args.steps * 1000.0
    if e2e_shard is not shard:
        torch.cuda.synchronize()
        if not torch.equal(yh, e2e_shard.y.cpu()):
            raise SystemExit("end-to-end result on the host differs from the device result")
        e2e_shard.destroy()
    io_bytes = args.batch * M.GPT3_HIDDEN * 2

    # ---- per-batch table ------------------------------------------------------------------------
    table = []
    if not args.no_sweep and world == 1:
        for b in SWEEP_BATCHES:
            row = {"batch": b}
            for pol in ("rowsync", "tilesync"):
                s = build(b, pol)

                def c_step(s=s):
                    s.run_cusync(ps, cs)

                def o_step(s=s):
                    s.run_stream_ordered(cs)

                c_per, o_per = interleaved(c_step, (ps, cs), o_step, (cs, cs), 20, 5)
                c_us, o_us = statistics.median(c_per) * 1000, statistics.median(o_per) * 1000
                row[pol + "_us"] = round(c_us, 2)
                row[pol + "_stream_ordered_us"] = round(o_us, 2)
                row[pol + "_gain_pct"] = round(100.0 - c_us / o_us * 100.0, 2)
                row["tile_n"] = [s.tile_n1, s.tile_n2]
                row["split_k"] = [s.split_k1, s.split_k2]
                row["single_grid"] = s.single_grid
                if s.status_codes() != (0, 0):
                    row["error"] = "bounded wait expired"
                if s.single_grid and pol == "rowsync":
                    # the reference-shaped form of the same layer: one launch per GEMM and a wait kernel
                    x2 = s.x; s.destroy()
                    s = M.MLPShard("gpt3", b, x2, s.w1, s.w2, None, policy=pol, single_grid=1)
                    c_per, o_per = interleaved(lambda s=s: s.run_cusync(ps, cs), (ps, cs),
                                               lambda s=s: s.run_stream_ordered(cs), (cs, cs), 20, 5)
                    row["rowsync_two_launches_us"] = round(statistics.median(c_per) * 1000, 2)
                s.destroy()
            # context only, as in the reference's tables (their "torch" column): the same layer through the vendor
            # library, y = gelu(x @ w1) @ w2 on one stream (cuBLAS GEMMs + an elementwise kernel), timed alike
            xs, w1s, w2s, _ = M.make_inputs("gpt3", b, dev, seed=rank)

            def t_step():
                with torch.cuda.stream(cs):
                    torch.matmul(torch.nn.functional.gelu(torch.matmul(xs, w1s)), w2s)
            t_per, _ = interleaved(t_step, (cs, cs), t_step, (cs, cs), 10, 3)
            row["torch_cublas_us"] = round(statistics.median(t_per) * 1000, 2)
            best = min(row["rowsync_us"], row["tilesync_us"], row["rowsync_stream_ordered_us"])
            row["tflops_best"] = round(shard.flops() / args.batch * b / (best * 1e-6) / 1e12, 1)
            table.append(row)
    # ---- the other workloads of the path: LLaMA MLP, 3x3 conv chain, attention block ------------------
    extras = {}
    if not args.no_sweep and world == 1:
        import cusync_b200 as lib_
        from cusync_b200.attention import AttentionBlock
        s3 = torch.cuda.Stream()

        def ab(c_step, o_step):
            c_per, o_per = interleaved(c_step, (ps, cs), o_step, (cs, cs), 20, 5)
            c_us, o_us = statistics.median(c_per) * 1000, statistics.median(o_per) * 1000
            return {"cusync_us": round(c_us, 2), "stream_ordered_us": round(o_us, 2),
                    "gain_pct": round(100.0 - c_us / o_us * 100.0, 2)}

        rows = []
        for b in (1, 64, 512, 2048):     # config 3: LLaMA 65B MLP shard, fused SwiGLU dual GEMM, ffn 2752
            x, w1, w2, v = M.make_inputs("llama", b, dev, seed=1)
            for pol in ("rowsync", "tilesync"):
                sh = M.MLPShard("llama", b, x, w1, w2, v, policy=pol)

                def c_step(sh=sh):
                    ps.wait_stream(cs); sh.run_cusync(ps, cs)
                r = ab(c_step, lambda sh=sh: sh.run_stream_ordered(cs))
                r.update({"batch": b, "policy": pol, "tile_n": [sh.tile_n1, sh.tile_n2],
                          "split_k": [sh.split_k1, sh.split_k2]})
                rows.append(r); sh.destroy()
        extras["llama_mlp"] = rows

        rows = []
        for n in (1, 8, 32):             # config 5: two 3x3 convolutions, 56x56x64, ReLU, Conv2DTileSync
            g = torch.Generator(device=dev).manual_seed(n)
            xin = torch.randn((n, 56, 56, 64), generator=g, device=dev).half()
            f1 = (torch.randn((64, 3, 3, 64), generator=g, device=dev) * (2.0 / 576) ** 0.5).half()
            f2 = (torch.randn((64, 3, 3, 64), generator=g, device=dev) * (2.0 / 576) ** 0.5).half()
            chain = lib_.ConvChain(xin, [f1, f2], relu=True)     # cusync_conv_chain_*: the resnet.cu flow in C

            def c_step():
                ps.wait_stream(cs); chain.run_cusync([ps, cs])

            def o_step():
                chain.run_stream_ordered(cs)
            r = ab(c_step, o_step)
            r["images"] = n
            r["wait_kernel"] = chain.uses_wait_kernels
            rows.append(r)
            chain.destroy()
        extras["resnet_conv3x3_chain_conv2dtilesync"] = rows

        # vgg.cu-style chain of four 64-channel convolutions, one stream per convolution
        g = torch.Generator(device=dev).manual_seed(44)
        xin = torch.randn((8, 56, 56, 64), generator=g, device=dev).half()
        fs = [(torch.randn((64, 3, 3, 64), generator=g, device=dev) * (2.0 / 576) ** 0.5).half() for _ in range(4)]
        chain = lib_.ConvChain(xin, fs, relu=True)
        side = [torch.cuda.Stream(), torch.cuda.Stream()]

        def c4_step():
            ps.wait_stream(cs); chain.run_cusync([ps, side[0], side[1], cs])

        def o4_step():
            chain.run_stream_ordered(cs)
        r = ab(c4_step, o4_step)
        r.update({"images": 8, "convs": 4})
        extras["vgg_conv3x3_chain_of_4"] = [r]
        chain.destroy()

        rows = []
        for b, seq in ((1, 512), (1, 2048), (4, 2048)):   # config 4: attention block, 12 heads of 128
            g = torch.Generator(device=dev).manual_seed(7)
            xin = torch.randn((b, 12288), generator=g, device=dev).half()
            wqkv = (torch.randn((12288, 4608), generator=g, device=dev) * 0.02).half()
            wo = (torch.randn((1536, 12288), generator=g, device=dev) * 0.02).half()
            kc = torch.randn((b, seq, 12, 128), generator=g, device=dev).half()
            vc = torch.randn((b, seq, 12, 128), generator=g, device=dev).half()
            blk = AttentionBlock(xin, wqkv, kc, vc, wo, 12)     # cusync_attn_block_*: the attention.cu flow in C

            def c_step():
                ps.wait_stream(s3); blk.run((ps, cs, s3)); cs.wait_stream(s3)
            r = ab(c_step, lambda: blk.run_stream_ordered(cs))
            r.update({"batch": b, "context": seq, "config": blk.config})
            rows.append(r); blk.destroy()
        extras["gpt3_attention_block"] = rows
    clocks = sampler.stop() if rank == 0 else None

    if rank != 0:
        group.close()
        return

    value_us = ms_per_step * 1000.0
    line = {"metric": METRIC, "value": value_us, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": False, "scaling": "weak",
            "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": workload_config(args, shard),
            "median_us": statistics.median(per_ms) * 1000.0,
            "stream_ordered_us": ord_ms * 1000.0,
            "gain_vs_stream_ordered_pct": 100.0 - ms_per_step / ord_ms * 100.0,
            "interleaved": {"cusync_us": il_c_us, "stream_ordered_us": il_o_us,
                            "gain_pct": 100.0 - il_c_us / il_o_us * 100.0,
                            "how": "arms alternated step by step, medians over %d steps each" % args.steps},
            "layer_tflops": shard.flops() / (ms_per_step * 1e-3) / 1e12,
            "layer_frac_of_sustained_peak": shard.flops() / (ms_per_step * 1e-3) / 1e12 / peaks["tflops_sustained"],
            "roofline": roofline,
            "e2e": {"value": e2e_us, "unit": UNIT, "h2d_bytes_per_step": io_bytes, "d2h_bytes_per_step": io_bytes},
            "gpu_launches": (1 if shard.single_grid else 3) * args.steps,
            "launch_form": ("one persistent grid for both GEMMs" if shard.single_grid
                            else "one launch per GEMM and a wait kernel"),
            "clocks": clocks,
            "per_batch": table,
            "other_workloads": extras}
    if not args.no_cpu:
        sample = args.batch
        us, threads, spent = cpu_reference_us(args.batch, sample, M.GPT3_HIDDEN, M.GPT3_FFN)
        line["cpu_baseline"] = {"value": us, "unit": UNIT, "cores": threads, "kind": "port",
                                "sample": "%d of %d rows through both GEMMs (%.1f s), scaled to the full batch"
                                          % (sample, args.batch, spent)}
    emit(line)
    group.close()


if __name__ == "__main__":
    main()
