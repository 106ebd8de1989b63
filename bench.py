#!/usr/bin/env python
"""Benchmark of the hot path: one GPT-3 175B MLP layer, one 8-way
tensor-parallel shard, as a chain of two tile-synchronised GEMMs.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch B] [--policy rowsync|tilesync]
    python bench.py --impl reference ...          # the CPU host-reference path, timed on the host cores

A step is one MLP layer over one batch of synthetic input (X ~ N(0,1),
weights ~ N(0,0.02), seeded): producer GEMM (+GELU) and consumer GEMM
synchronised tile by tile through semaphores (one launch each with a wait
kernel, or one persistent grid for both, as the library's table picks); with
N > 1 GPUs the sum all-reduce of the [B, 12288] output runs as this library's
kernel beside the second GEMM (--reduce nccl: NCCL's all-reduce after it).
One JSON line is printed by rank 0.  Time-like metric: microseconds per layer.
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

    def __init__(self, index, period_ms=100):
        self.index, self.rows, self.proc, self.period_ms = index, [], None, period_ms

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", str(self.period_ms)],
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


def host_threads():
    """Threads the CPU arm uses: every core this process may run on (a launcher such as torchrun exports
    OMP_NUM_THREADS=1 to its workers, which is not what a host-side baseline should inherit)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def cpu_reference_us(batch, sample_rows, hidden, ffn):
    """The CPU host-reference path (oracle restatement of ref_cpumatmul + GELU) on `sample_rows` rows of the
    layer, all host threads; returns (microseconds scaled to `batch` rows, threads, seconds spent)."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import numpy as np
    import oracle_lib as o
    o.set_num_threads(host_threads())
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
    restatement of ref_cpumatmul (kind "port").  Rank 0 alone runs it; a step is a bounded sample of the layer
    (512 of its rows through both GEMMs, scaled to the batch) and at most three steps are timed, so the arm ends
    within a minute whatever --steps says."""
    if rank != 0:
        return
    os.environ["OMP_NUM_THREADS"] = str(host_threads())
    from cusync_b200 import mlp as M
    hidden, ffn = M.GPT3_HIDDEN, M.GPT3_FFN
    sample = min(args.batch, 512)
    steps, warmup = min(args.steps, 3), min(args.warmup, 1)
    times = []
    for i in range(warmup + steps):
        us, threads, _ = cpu_reference_us(args.batch, sample, hidden, ffn)
        if i >= warmup:
            times.append(us)
    val = statistics.mean(times)
    line = {"impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus,
            "steps": steps, "warmup": warmup, "ms_per_step": val / 1000.0, "higher_is_better": False,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": workload_config(args, None),
            "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "kind": "port",
                             "sample": "%d of %d rows through both GEMMs, scaled to the full batch; %d timed steps"
                                       % (sample, args.batch, steps)},
            "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    emit(line)


def workload_config(args, shard):
    cfg = {"workload": "GPT-3 175B MLP, one 8-way tensor-parallel shard: X[%d,12288] * W1[12288,6144] -> GELU -> "
                       "* W2[6144,12288]" % args.batch,
           "batch": args.batch, "policy": args.policy,
           "l2": "inputs larger than L2 (302 MB of weights per step vs 126 MB L2); no explicit flush",
           "all_reduce": (("sum of Y[B,12288] fp16 across ranks by this library's kernel beside the second GEMM "
                           "(%d blocks; the GEMMs use the other SMs)" % (args.reduce_ctas if args.reduce_ctas > 0 else 4)
                           if getattr(args, "reduce", "overlapped") == "overlapped" and args.batch >= 1024
                           else "NCCL sum of Y[B,12288] fp16 across ranks, after the layer")
                          if args.gpus > 1 else "none (1 GPU)")}
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


def load_traffic(kernel_key, batch):
    """dram__bytes_read.sum + dram__bytes_write.sum of one launch, as captured with ncu (bytes), or None."""
    path = os.path.join(ROOT, "profiles", "dram_traffic.json")
    try:
        table = json.load(open(path))
    except (OSError, ValueError):
        return None
    for key, per_batch in table.items():
        if key.startswith(kernel_key) and isinstance(per_batch, dict):
            return per_batch.get(str(batch))
    return None


def overlap_timeline(shard, ps, cs):
    """What the consumer GEMM's tiles do while the producer's last tiles still run, from one traced run of the
    synchronised layer (the per-tile timeline of the CTA-pair kernels): the evidence a profiler cannot give,
    since it serialises the two kernels."""
    import numpy as np
    for _ in range(3):
        shard.run_cusync(ps, cs)
    best = None
    for _ in range(3):                           # the quickest of three traced runs (the clock drifts between runs)
        t1, t2 = shard.traced_run(ps, cs)
        a, b = t1[0::2], t2[0::2]                # the leader CTA's record of every work unit
        a, b = a[a[:, 0] > 0], b[b[:, 0] > 0]
        if len(a) == 0 or len(b) == 0:
            return None
        span = int(b[:, 2].max()) - int(a[:, 0].min())
        if best is None or span < best[0]:
            best = (span, a, b)
    g1, g2 = best[1], best[2]
    t0 = int(g1[:, 0].min())
    p_last_draw, p_end = int(g1[:, 0].max()), int(g1[:, 2].max())
    early = g2[g2[:, 0] < p_end]
    late = g2[g2[:, 0] >= p_end]

    def part(rs):
        if len(rs) == 0:
            return None
        cyc = float(rs[:, 6].sum())
        return {"units": int(len(rs)), "mma_thread_cycles_per_unit": round(cyc / len(rs)),
                "waiting_for_operands_pct": round(100.0 * float(rs[:, 4].sum()) / cyc, 1),
                "waiting_for_accumulator_pct": round(100.0 * float(rs[:, 7].sum()) / cyc, 1),
                "loader_waiting_for_ring_slot_pct": round(100.0 * float(rs[:, 5].sum()) / cyc, 1),
                "wall_us_per_unit": round(float((rs[:, 2] - rs[:, 0]).mean()) / 1e3, 1)}
    return {"launch_form": "one persistent grid" if shard.single_grid else "one launch per GEMM and a wait kernel",
            "producer_units": int(len(g1)), "consumer_units": int(len(g2)),
            "producer_last_draw_us": round((p_last_draw - t0) / 1e3, 1), "producer_end_us": round((p_end - t0) / 1e3, 1),
            "consumer_first_draw_us": round((int(g2[:, 0].min()) - t0) / 1e3, 1),
            "consumer_end_us": round((int(g2[:, 2].max()) - t0) / 1e3, 1),
            "consumer_units_drawn_before_producer_end": int(len(early)),
            "consumer_units_finished_before_producer_end": int((g2[:, 2] < p_end).sum()),
            "pairs_on_consumer_units_before_producer_end": int(len(np.unique(early[:, 3] & 0xffffffff))),
            "producer": part(g1), "consumer_drawn_before_producer_end": part(early),
            "consumer_drawn_after_producer_end": part(late)}


def main():
    _watchdog(1500)
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=2048)
    ap.add_argument("--policy", default="rowsync", choices=["rowsync", "tilesync", "auto"])
    ap.add_argument("--impl", default="cusync", choices=["cusync", "reference"])
    ap.add_argument("--reduce", choices=("overlapped", "nccl"), default="overlapped",
                    help="multi-GPU: the all-reduce of Y as this library's kernel beside the second GEMM (default), "
                         "or NCCL's all-reduce after the layer")
    ap.add_argument("--reduce-ctas", type=int, default=0,
                    help="blocks of the overlapped all-reduce kernel (0 = choose: 4, which leaves the GEMMs 72 SM pairs: "
                         "the 576 pair tiles of the B = 2048 layer are then exactly eight rounds)")
    ap.add_argument("--no-sweep", action="store_true", help="skip the per-batch table and the other workloads")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--group-rows1", type=int, default=0, help="tile order of the first GEMM (0 = the library's table)")
    ap.add_argument("--group-rows2", type=int, default=0, help="tile order of the second GEMM (0 = the library's table)")
    ap.add_argument("--timeline", action="store_true",
                    help="add `overlap_timeline`: one traced run of the layer in both launch forms (per-tile timeline)")
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
    sms = torch.cuda.get_device_properties(dev).multi_processor_count

    def barrier():
        group.barrier()

    def reduce_max(v):
        return group.max_over_ranks(v)

    peaks = load_peaks()
    ps = torch.cuda.Stream(priority=-1)   # producer: high priority, launched first
    cs = torch.cuda.Stream(priority=0)
    rs = torch.cuda.Stream(priority=0)    # multi-GPU: the all-reduce kernel that runs beside the GEMMs
    overlap_reduce = world > 1 and args.reduce == "overlapped"
    if args.reduce_ctas <= 0:
        args.reduce_ctas = 4
    # The all-reduce kernel hides behind the second GEMM where that GEMM runs longer than the exchange takes on a
    # few SMs: the GPT-3 shard from eight row tiles on (measured on 2 GPUs: +4.6 % at B = 1024, +10 % at 2048, -1 %
    # at 512).  Elsewhere (small batches; the LLaMA shard, whose second GEMM is short) NCCL's all-reduce after
    # the layer is the better form.
    OVERLAP_MIN_BATCH = 1024

    class Layer:
        """One tensor-parallel layer of `model` at `batch`: the synchronised chain with its all-reduce (this
        library's kernel beside the GEMMs, or NCCL after them) and the same kernels stream-ordered with NCCL."""

        def __init__(self, model, batch, policy, seed):
            x, w1, w2, v = M.make_inputs(model, batch, dev, seed=seed)
            self.model, self.batch = model, batch
            self.reducer = None
            if overlap_reduce and batch >= OVERLAP_MIN_BATCH and model == "gpt3":
                self.reducer = tp.RowAllReduce(group, batch, x.shape[1], dev, num_ctas=args.reduce_ctas)
                self.shard = M.MLPShard(model, batch, x, w1, w2, v, policy=policy, post_rows=True,
                                        max_ctas=sms - self.reducer.num_ctas, y=self.reducer.y)
                # the stream-ordered arm keeps the whole device and its own output
                self.base = M.MLPShard(model, batch, x, w1, w2, v, policy=policy, single_grid=1)
            else:
                self.shard = M.MLPShard(model, batch, x, w1, w2, v, policy=policy, group_rows1=args.group_rows1,
                                        group_rows2=args.group_rows2)
                self.base = self.shard

        def cusync_step(self):
            if self.reducer is not None:
                self.shard.run_cusync_allreduce(self.reducer, ps, cs, rs)
            else:
                self.shard.run_cusync(ps, cs)
                if world > 1:
                    with torch.cuda.stream(cs):
                        group.all_reduce_sum(self.shard.y)

        def chain_only_step(self):
            """The layer without its all-reduce (what one GPU runs)."""
            self.base.run_cusync(ps, cs)

        def ordered_step(self):
            self.base.run_stream_ordered(cs)
            if world > 1:
                with torch.cuda.stream(cs):
                    group.all_reduce_sum(self.base.y)

        def check(self):
            """The overlapped all-reduce gives what NCCL's all-reduce of the same partial outputs gives, up to the
            order of the sum: this library's kernel adds the ranks' fp16 values in fp32 and rounds once."""
            if self.reducer is None:
                return None
            self.cusync_step(); torch.cuda.synchronize(); barrier()
            self.ordered_step(); torch.cuda.synchronize(); barrier()
            ref, got = self.base.y.float(), self.shard.y.float()
            err = (got - ref).abs().max().item() / max(ref.abs().max().item(), 1e-6)
            if not err <= 4e-3:
                raise SystemExit("overlapped all-reduce differs from NCCL's: %.3e of max|Y|" % err)
            return err

        def status_ok(self):
            ok = self.shard.status_codes() == (0, 0)
            return ok and (self.reducer is None or self.reducer.status_code() == 0)

        def destroy(self):
            if self.base is not self.shard:
                self.base.destroy()
            self.shard.destroy()
            if self.reducer is not None:
                self.reducer.destroy()

    layer = Layer("gpt3", args.batch, args.policy, seed=rank)
    shard = layer.shard
    reduce_err = layer.check()

    side_streams = []          # every further stream an arm launches on registers here

    def interleaved_arms(arms, n, warm):
        """Alternates the arms [(step, (first stream, last stream)), ...] step by step, so clock and power drift
        hits all alike.  Before every step all streams meet: the arm's first stream waits for everything
        enqueued so far and every other stream waits for that point, so that no kernel of a step (a consumer on a
        side stream, say) can become resident while the previous step of another arm still runs.
        Returns one per-step millisecond list per arm."""
        streams = [ps, cs, rs] + side_streams
        for _ in range(warm):
            for fn, _ in arms:
                fn()
        torch.cuda.synchronize()
        barrier()
        ev = [[] for _ in arms]
        for _ in range(n):
            for i, (fn, (s0, s1)) in enumerate(arms):
                for s in streams:
                    if s is not s0:
                        s0.wait_stream(s)
                for s in streams:
                    if s is not s0:
                        s.wait_stream(s0)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(s0); fn(); e1.record(s1)
                ev[i].append((e0, e1))
        torch.cuda.synchronize()
        return [[a.elapsed_time(b) for a, b in e] for e in ev]

    def interleaved(step_a, a_streams, step_b, b_streams, n, warm):
        return interleaved_arms([(step_a, a_streams), (step_b, b_streams)], n, warm)

    def med_us(ms_list):
        return reduce_max(statistics.median(ms_list) * 1000.0)

    # ---- headline: overlapped chain ------------------------------------------------------------
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    total_ms, per_ms = time_steps(layer.cusync_step, ps, cs, args.steps, args.warmup, barrier)
    total_ms = reduce_max(total_ms)
    ms_per_step = total_ms / args.steps
    if not layer.status_ok():
        raise SystemExit("a bounded wait expired during the timed region")

    # ---- same kernels serialised by stream order --------------------------------------------
    ord_total, ord_per = time_steps(layer.ordered_step, cs, cs, args.steps, args.warmup, barrier)
    ord_ms = reduce_max(ord_total) / args.steps
    # ... and both arms interleaved step by step (the fair comparison under clock drift)
    il_c, il_o = interleaved(layer.cusync_step, (ps, cs), layer.ordered_step, (cs, cs), args.steps, 3)
    il_c_us, il_o_us = med_us(il_c), med_us(il_o)

    # ---- multi-GPU: the layer without its all-reduce, and the all-reduce alone ---------------------------
    multi = None
    if world > 1:
        def chain_vs_layer():
            c_per, l_per = interleaved(layer.chain_only_step, (ps, cs), layer.cusync_step, (ps, cs), args.steps, 3)
            return med_us(c_per), med_us(l_per)

        def allreduce_alone(buf, n):
            """The isolated collective on the layer's output buffer: barrier, then n back-to-back all-reduces
            between one pair of events (the protocol of allreduce_times.py:13-28)."""
            for _ in range(3):
                with torch.cuda.stream(cs):
                    group.all_reduce_sum(buf)
            torch.cuda.synchronize(); barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            with torch.cuda.stream(cs):
                e0.record(cs)
                for _ in range(n):
                    group.all_reduce_sum(buf)
                e1.record(cs)
            torch.cuda.synchronize()
            return reduce_max(e0.elapsed_time(e1) / n * 1000.0)

        def own_allreduce_alone(reducer, n):
            if reducer is None:
                return None
            for _ in range(3):
                reducer.run(rs)
            torch.cuda.synchronize(); barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(rs)
            for _ in range(n):
                reducer.run(rs)
            e1.record(rs)
            torch.cuda.synchronize()
            return reduce_max(e0.elapsed_time(e1) / n * 1000.0)

        chain_us, layer_us = chain_vs_layer()
        # for comparison: the synchronised chain on the whole device, NCCL's all-reduce after it
        def nccl_after_step():
            layer.base.run_cusync(ps, cs)
            with torch.cuda.stream(cs):
                group.all_reduce_sum(layer.base.y)
        na_per, _ = interleaved(nccl_after_step, (ps, cs), layer.ordered_step, (cs, cs), args.steps, 3)
        multi = {"layer_without_allreduce_us": chain_us, "layer_with_allreduce_us": layer_us,
                 "cusync_chain_then_nccl_allreduce_us": med_us(na_per),
                 "allreduce_alone_us": allreduce_alone(layer.base.y, 20),
                 "own_allreduce_kernel_alone_us": own_allreduce_alone(layer.reducer, 20),
                 "allreduce_form": ("this library's kernel beside the second GEMM: %d blocks, %s, GEMMs on %d of %d SMs"
                                    % (layer.reducer.num_ctas,
                                       "multimem.ld_reduce / multimem.st through the NVSwitch" if layer.reducer.uses_multicast
                                       else "peer loads and stores", sms - layer.reducer.num_ctas, sms))
                                   if layer.reducer is not None else "NCCL all-reduce after the layer",
                 "overlapped_vs_nccl_max_err_of_max": reduce_err, "per_batch": []}
        if not args.no_sweep:
            for b in SWEEP_BATCHES:
                lb = Layer("gpt3", b, args.policy, seed=rank)
                lb.check()
                c_per, l_per = interleaved(lb.chain_only_step, (ps, cs), lb.cusync_step, (ps, cs), 20, 3)
                l2_per, o_per = interleaved(lb.cusync_step, (ps, cs), lb.ordered_step, (cs, cs), 20, 3)
                multi["per_batch"].append({
                    "batch": b, "layer_without_allreduce_us": round(med_us(c_per), 2),
                    "layer_with_allreduce_us": round(med_us(l_per), 2),
                    "stream_ordered_with_nccl_us": round(med_us(o_per), 2),
                    "gain_pct": round(100.0 - med_us(l2_per) / med_us(o_per) * 100.0, 2),
                    "allreduce_alone_us": round(allreduce_alone(lb.base.y, 20), 2),
                    "own_allreduce_kernel_alone_us": (round(own_allreduce_alone(lb.reducer, 20), 2)
                                                      if lb.reducer is not None else None)})
                if not lb.status_ok():
                    multi["per_batch"][-1]["error"] = "bounded wait expired"
                lb.destroy()

    timeline = None
    if args.timeline and world == 1 and args.batch > 256:
        timeline = []
        for sg in (2, 1):
            ts = M.MLPShard("gpt3", args.batch, shard.x, shard.w1, shard.w2, None, policy=args.policy, single_grid=sg)
            timeline.append(overlap_timeline(ts, ps, cs))
            ts.destroy()

    # ---- per-kernel durations: each GEMM alone and both in a row, back to back between ONE pair of events ----
    base = layer.base
    flops2 = 2.0 * args.batch * M.GPT3_FFN * M.GPT3_HIDDEN
    loop_n = max(200, args.steps)

    def loop_ms(fn, n):
        for _ in range(max(args.warmup, 3)):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(cs)
        for _ in range(n):
            fn()
        e1.record(cs)
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    kernel_clock = ClockSampler(local_rank, period_ms=20)
    if rank == 0:
        kernel_clock.start()
    t2_ms = loop_ms(lambda: base.run_single(2, cs), loop_n)
    t1_ms = loop_ms(lambda: base.run_single(1, cs), loop_n)
    t12_ms = loop_ms(lambda: base.run_stream_ordered(cs), loop_n)
    kclk = kernel_clock.stop() if rank == 0 else {"sm_mhz": None}
    traffic = load_traffic("cusync_gemm_pair_kernel GEMM2", args.batch) if args.batch > 256 else None
    tensor_bound = args.batch >= 256
    kernel_name = ("cusync_gemm_pair_kernel (GEMM2, the consumer)" if args.batch > 256
                   else "cusync_gemm_kernel<%d,0> (GEMM2, the consumer)" % shard.tile_n2)
    mhz = kclk.get("sm_mhz")
    timing = {"launch_ms": t2_ms, "gemm1_ms": t1_ms, "both_in_a_row_ms": t12_ms,
              "sum_of_the_two_over_both_in_a_row": (t1_ms + t2_ms) / t12_ms,
              "launches_per_loop": loop_n, "sm_mhz_during_loops": mhz,
              "launch_ms_x_mhz": t2_ms * mhz if mhz else None,
              "how": "each figure = %d launches back to back between one pair of events on the launching stream; the "
                     "three loops run one after the other under one clock sampler" % loop_n}
    if tensor_bound:
        achieved = flops2 / (t2_ms * 1e-3) / 1e12
        roofline = {"bound": "tensor", "kernel": kernel_name, "achieved": achieved, "peak": peaks["tflops_burst"],
                    "unit": "TFLOP/s", "frac": achieved / peaks["tflops_burst"],
                    "peak_kind": "%s burst bf16/fp16 cuBLAS figure (the kernel is timed alone)" % peaks["source"],
                    "frac_of_sustained_peak": achieved / peaks["tflops_sustained"], "traffic": traffic,
                    "gemm1_tflops": flops2 / (t1_ms * 1e-3) / 1e12}
    else:
        bytes2 = 2.0 * (M.GPT3_FFN * M.GPT3_HIDDEN + args.batch * (M.GPT3_FFN + M.GPT3_HIDDEN))
        achieved = bytes2 / (t2_ms * 1e-3) / 1e9
        roofline = {"bound": "hbm", "kernel": kernel_name, "achieved": achieved, "peak": peaks["hbm_gbs"],
                    "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                    "peak_kind": "%s copy bandwidth" % peaks["source"], "traffic": traffic}
    roofline.update(timing)

    # ---- end to end through the C ABI with host buffers ---------------------------------------
    xh = torch.empty((args.batch, M.GPT3_HIDDEN), dtype=torch.half).pin_memory()
    xh.copy_(shard.x.cpu())
    yh = torch.empty((args.batch, M.GPT3_HIDDEN), dtype=torch.half).pin_memory()

    # One GPU: the result goes back to the host in row blocks, each behind the RowSync semaphores of its 128-row
    # tiles of the second GEMM (post_rows), so the device-to-host copy overlaps that GEMM.  Each GEMM gets half of
    # the SMs here: a persistent kernel that holds every SM while it waits for rows of X keeps the second GEMM
    # from becoming resident, and with it the first rows of Y from leaving while the last rows of X arrive.  The
    # step is bound by the PCIe link, not by the GEMMs, so halving their rate costs nothing.
    e2e_shard, e2e_reducer = shard, None
    d2h_blocks = 4
    row_blocks = args.batch >= 512
    if row_blocks:
        d2h_blocks = max(4, min(8, args.batch // 256))
        if world == 1:
            e2e_ctas = sms // 4 * 2
            e2e_shard = M.MLPShard("gpt3", args.batch, shard.x, shard.w1, shard.w2, None, policy=args.policy,
                                   post_rows=True, x_rows=True, max_ctas=e2e_ctas, group_rows2=2, single_grid=1)
        else:
            # N > 1: X is replicated over the ranks and Y is the same on all of them after the all-reduce, so the job
            # moves each of them over PCIe ONCE: rank r fetches rows [r, r + 1) * B / N of X from the host, an
            # all-gather over NVLink completes X everywhere, and rank r returns its B / N rows of Y.
            if overlap_reduce and args.batch >= OVERLAP_MIN_BATCH:
                e2e_reducer = tp.RowAllReduce(group, args.batch, M.GPT3_HIDDEN, dev, num_ctas=args.reduce_ctas)
            e2e_shard = M.MLPShard("gpt3", args.batch, shard.x, shard.w1, shard.w2, None, policy=args.policy,
                                   post_rows=e2e_reducer is not None,
                                   max_ctas=sms - (e2e_reducer.num_ctas if e2e_reducer else 0),
                                   y=e2e_reducer.y if e2e_reducer else None)
    d2h, h2d, post = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    landed = [torch.cuda.Event() for _ in range(d2h_blocks)]

    share = args.batch // world if args.batch % world == 0 else 0     # rows of X and of Y this rank moves (N > 1)

    def e2e_step_sharded():
        r0, r1 = rank * share, (rank + 1) * share
        with torch.cuda.stream(ps):
            e2e_shard.x[r0:r1].copy_(xh[r0:r1], non_blocking=True)
            group.all_gather_rows(e2e_shard.x, share)
        if e2e_reducer is not None:
            e2e_shard.run_cusync_allreduce(e2e_reducer, ps, cs, rs)
        else:
            e2e_shard.run_cusync(ps, cs)
            with torch.cuda.stream(cs):
                group.all_reduce_sum(e2e_shard.y)
        with torch.cuda.stream(cs):
            yh[r0:r1].copy_(e2e_shard.y[r0:r1], non_blocking=True)

    def e2e_step():
        if world > 1 and share > 0 and row_blocks:
            return e2e_step_sharded()
        tiles = (args.batch + 127) // 128
        per = (tiles + d2h_blocks - 1) // d2h_blocks
        if row_blocks:
            # X comes in row blocks on its own stream, each followed by the post of its RowSync semaphores; the
            # first GEMM is launched right away and takes the rows as they land (x_rows)
            h2d.wait_stream(cs)
            post.wait_stream(cs)
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
        if e2e_reducer is not None:
            e2e_shard.run_cusync_allreduce(e2e_reducer, ps, cs, rs)
        else:
            e2e_shard.run_cusync(ps, cs)
        if row_blocks and world == 1:
            for first in range(0, tiles, per):
                n = min(per, tiles - first)
                e2e_shard.wait_rows(first, n, d2h)
                r0, r1 = first * 128, min(args.batch, (first + n) * 128)
                with torch.cuda.stream(d2h):
                    yh[r0:r1].copy_(e2e_shard.y[r0:r1], non_blocking=True)
            cs.wait_stream(d2h)
        else:
            with torch.cuda.stream(cs):
                if world > 1 and e2e_reducer is None:
                    group.all_reduce_sum(e2e_shard.y)
                yh.copy_(e2e_shard.y, non_blocking=True)

    e2e_total, _ = time_steps(e2e_step, ps, cs, args.steps, args.warmup, barrier)
    e2e_us = reduce_max(e2e_total) / args.steps * 1000.0
    if e2e_shard is not shard:
        torch.cuda.synchronize()
        lo, hi = (rank * share, (rank + 1) * share) if (world > 1 and share > 0) else (0, args.batch)
        if not torch.equal(yh[lo:hi], e2e_shard.y[lo:hi].cpu()):
            raise SystemExit("end-to-end result on the host differs from the device result")
        e2e_shard.destroy()
        if e2e_reducer is not None:
            e2e_reducer.destroy()
    io_bytes = args.batch * M.GPT3_HIDDEN * 2       # whole job: at N > 1 every rank moves 1 / N of it each way

    # ---- per-batch table ------------------------------------------------------------------------
    table = []
    if not args.no_sweep and world == 1:
        for b in SWEEP_BATCHES:
            row = {"batch": b}
            for pol in ("rowsync", "tilesync"):
                s = M.MLPShard("gpt3", b, *M.make_inputs("gpt3", b, dev, seed=rank), policy=pol)

                def c_step(s=s):
                    s.run_cusync(ps, cs)

                def o_step(s=s):
                    s.run_stream_ordered(cs)

                c_per, o_per = interleaved(c_step, (ps, cs), o_step, (cs, cs), 20, 5)
                c_us, o_us = statistics.median(c_per) * 1000, statistics.median(o_per) * 1000
                row[pol + "_us"] = round(c_us, 2)
                row[pol + "_stream_ordered_us"] = round(o_us, 2)
                row[pol + "_gain_pct"] = round(100.0 - c_us / o_us * 100.0, 2)
                if pol == "rowsync" and not s.single_grid:
                    # the two synchronised launches on ONE stream, the consumer a programmatic dependent launch
                    d_per, o2_per = interleaved(lambda s=s: s.run_dependent(cs), (cs, cs), o_step, (cs, cs), 20, 5)
                    row["rowsync_dependent_launch_us"] = round(statistics.median(d_per) * 1000, 2)
                    row["rowsync_dependent_launch_gain_pct"] = round(
                        100.0 - statistics.median(d_per) / statistics.median(o2_per) * 100.0, 2)
                row["tile_n"] = [s.tile_n1, s.tile_n2]
                row["split_k"] = [s.split_k1, s.split_k2]
                row["single_grid"] = s.single_grid
                if s.status_codes() != (0, 0):
                    row["error"] = "bounded wait expired"
                if s.single_grid and pol == "rowsync":
                    # the reference-shaped form of the same layer: one launch per GEMM and a wait kernel
                    x2 = s.x; s.destroy()
                    s = M.MLPShard("gpt3", b, x2, s.w1, s.w2, None, policy=pol, single_grid=1)
                    c_per, o_per, d_per = interleaved_arms([(lambda s=s: s.run_cusync(ps, cs), (ps, cs)),
                                                            (lambda s=s: s.run_stream_ordered(cs), (cs, cs)),
                                                            (lambda s=s: s.run_dependent(cs), (cs, cs))], 20, 5)
                    o2 = statistics.median(o_per)
                    row["rowsync_two_launches_us"] = round(statistics.median(c_per) * 1000, 2)
                    row["rowsync_two_launches_gain_pct"] = round(100.0 - statistics.median(c_per) / o2 * 100.0, 2)
                    row["rowsync_dependent_launch_us"] = round(statistics.median(d_per) * 1000, 2)
                    row["rowsync_dependent_launch_gain_pct"] = round(100.0 - statistics.median(d_per) / o2 * 100.0, 2)
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
        side_streams.append(s3)

        def ab(c_step, o_step, d_step=None):
            """Stream form (the reference's: one stream per stage) against the stream-ordered arm and, where
            given, the one-stream form whose dependent stages are programmatic dependent launches."""
            arms = [(c_step, (ps, cs)), (o_step, (cs, cs))] + ([(d_step, (cs, cs))] if d_step else [])
            per = interleaved_arms(arms, 20, 5)
            c_us, o_us = statistics.median(per[0]) * 1000, statistics.median(per[1]) * 1000
            r = {"cusync_us": round(c_us, 2), "stream_ordered_us": round(o_us, 2),
                 "gain_pct": round(100.0 - c_us / o_us * 100.0, 2)}
            if d_step:
                d_us = statistics.median(per[2]) * 1000
                r["dependent_launch_us"] = round(d_us, 2)
                r["dependent_launch_gain_pct"] = round(100.0 - d_us / o_us * 100.0, 2)
            return r

        rows = []
        for b in (1, 64, 512, 2048):     # config 3: LLaMA 65B MLP shard, fused SwiGLU dual GEMM, ffn 2752
            x, w1, w2, v = M.make_inputs("llama", b, dev, seed=1)
            for pol in ("rowsync", "tilesync"):
                sh = M.MLPShard("llama", b, x, w1, w2, v, policy=pol)

                r = ab(lambda sh=sh: sh.run_cusync(ps, cs), lambda sh=sh: sh.run_stream_ordered(cs),
                       (lambda sh=sh: sh.run_dependent(cs)) if pol == "rowsync" else None)
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
                chain.run_cusync([ps, cs])

            def o_step():
                chain.run_stream_ordered(cs)
            r = ab(c_step, o_step, lambda: chain.run_dependent(cs))
            r["images"] = n
            r["wait_kernel"] = chain.uses_wait_kernels
            rows.append(r)
            chain.destroy()
        extras["resnet_conv3x3_chain_conv2dtilesync"] = rows

        # the reference's other layer sizes (eval_resnet.py:12-17, 497-498): 128 / 256 / 512 channels on
        # 28x28 / 14x14 / 7x7 images, two convolutions, general implicit-GEMM kernel
        rows = []
        for c, hw_ in ((128, 28), (256, 14), (512, 7)):
            for n in (8, 32):
                g = torch.Generator(device=dev).manual_seed(c + n)
                xin = torch.randn((n, hw_, hw_, c), generator=g, device=dev).half()
                fs = [(torch.randn((c, 3, 3, c), generator=g, device=dev) * (2.0 / (9 * c)) ** 0.5).half() for _ in range(2)]
                chain = lib_.ConvChain(xin, fs, relu=True)
                r = ab(lambda chain=chain: chain.run_cusync([ps, cs]), lambda chain=chain: chain.run_stream_ordered(cs),
                       lambda chain=chain: chain.run_dependent(cs))
                r.update({"channels": c, "image": hw_, "images": n, "wait_kernel": chain.uses_wait_kernels,
                          "tflops": round(2 * 2.0 * n * hw_ * hw_ * c * 9 * c / (r["cusync_us"] * 1e-6) / 1e12, 1)})
                rows.append(r)
                chain.destroy()
        extras["resnet_conv3x3_chain_other_layers"] = rows

        # vgg.cu-style chain of four 64-channel convolutions, one stream per convolution
        g = torch.Generator(device=dev).manual_seed(44)
        xin = torch.randn((8, 56, 56, 64), generator=g, device=dev).half()
        fs = [(torch.randn((64, 3, 3, 64), generator=g, device=dev) * (2.0 / 576) ** 0.5).half() for _ in range(4)]
        chain = lib_.ConvChain(xin, fs, relu=True)
        side = [torch.cuda.Stream(), torch.cuda.Stream()]
        side_streams.extend(side)

        def c4_step():
            chain.run_cusync([ps, side[0], side[1], cs])

        def o4_step():
            chain.run_stream_ordered(cs)
        r = ab(c4_step, o4_step, lambda: chain.run_dependent(cs))
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
                blk.run((ps, cs, s3)); cs.wait_stream(s3)
            r = ab(c_step, lambda: blk.run_stream_ordered(cs), lambda: blk.run_dependent(cs))
            r.update({"batch": b, "context": seq, "config": blk.config})
            rows.append(r); blk.destroy()
        extras["gpt3_attention_block"] = rows
        # the attention block in the prompt phase, as the reference runs it (attention.cu:272-276, seqlen = 0):
        # XQKV = X Wqkv; S = Q K^T; O = S V; Y = O Wo, four GEMMs on four streams.  X ~ N(0, 0.1^2) keeps O in fp16.
        from cusync_b200.attention import PromptAttentionBlock
        s4 = torch.cuda.Stream()
        side_streams.append(s4)
        rows = []
        for b in (512, 1024, 2048):
            g = torch.Generator(device=dev).manual_seed(9)
            xin = (torch.randn((b, 12288), generator=g, device=dev) * 0.1).half()
            wqkv = (torch.randn((12288, 4608), generator=g, device=dev) * 0.02).half()
            wo = (torch.randn((1536, 12288), generator=g, device=dev) * 0.02).half()
            blk = PromptAttentionBlock(xin, wqkv, wo, 12)

            def c_step(blk=blk):
                blk.run((ps, s3, s4, cs))
            r = ab(c_step, lambda blk=blk: blk.run_stream_ordered(cs), lambda blk=blk: blk.run_dependent(cs))
            r.update({"batch": b, "tflops": round(blk.flops() / (r["cusync_us"] * 1e-6) / 1e12, 1),
                      "ok": blk.status_codes() == (0, 0, 0, 0)})
            rows.append(r); blk.destroy()
        extras["gpt3_attention_prompt_phase"] = rows
    if not args.no_sweep and world > 1:
        # the other sharded workloads at N GPUs: LLaMA MLP shard (config 3) with the overlapped all-reduce, and the
        # attention block (config 4: 12 of 96 heads per rank) with NCCL's all-reduce of its output after the chain
        from cusync_b200.attention import AttentionBlock
        s3 = torch.cuda.Stream()
        side_streams.append(s3)
        rows = []
        for b in (64, 512, 2048):
            lb = Layer("llama", b, "rowsync", seed=rank)
            lb.check()
            c_per, o_per = interleaved(lb.cusync_step, (ps, cs), lb.ordered_step, (cs, cs), 20, 3)
            n_per, l_per = interleaved(lb.chain_only_step, (ps, cs), lb.cusync_step, (ps, cs), 20, 3)
            rows.append({"batch": b, "cusync_us": round(med_us(c_per), 2), "stream_ordered_us": round(med_us(o_per), 2),
                         "gain_pct": round(100.0 - med_us(c_per) / med_us(o_per) * 100.0, 2),
                         "layer_without_allreduce_us": round(med_us(n_per), 2), "ok": lb.status_ok()})
            lb.destroy()
        extras["llama_mlp"] = rows
        rows = []
        for b, seq in ((1, 2048), (4, 2048)):
            g = torch.Generator(device=dev).manual_seed(7 + rank)
            xin = torch.randn((b, 12288), generator=g, device=dev).half()
            wqkv = (torch.randn((12288, 4608), generator=g, device=dev) * 0.02).half()
            wo = (torch.randn((1536, 12288), generator=g, device=dev) * 0.02).half()
            kc = torch.randn((b, seq, 12, 128), generator=g, device=dev).half()
            vc = torch.randn((b, seq, 12, 128), generator=g, device=dev).half()
            blk = AttentionBlock(xin, wqkv, kc, vc, wo, 12)

            def c_step():
                blk.run((ps, cs, s3)); cs.wait_stream(s3)
                with torch.cuda.stream(cs):
                    group.all_reduce_sum(blk.y)

            def o_step():
                blk.run_stream_ordered(cs)
                with torch.cuda.stream(cs):
                    group.all_reduce_sum(blk.y)
            c_per, o_per = interleaved(c_step, (ps, cs), o_step, (cs, cs), 20, 3)
            rows.append({"batch": b, "context": seq, "cusync_us": round(med_us(c_per), 2),
                         "stream_ordered_us": round(med_us(o_per), 2),
                         "gain_pct": round(100.0 - med_us(c_per) / med_us(o_per) * 100.0, 2),
                         "all_reduce": "NCCL, after the output projection"})
            blk.destroy()
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
            "multi_gpu": multi,
            "overlap_timeline": timeline,
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
