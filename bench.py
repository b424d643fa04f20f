#!/usr/bin/env python
"""Benchmark of the sampling hot path: sampled edges/s on products-scale 3-hop GraphSAGE sampling.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (config "products-scale GraphSAGE 3-hop"): symmetric R-MAT graph, 2,450,000 nodes, 123,700,000 directed
edges, int64 CSC, hub degrees thinned to about 17k; train split = 8% of the nodes; minibatches of 1,024 seeds; per hop
(fanouts 15, 10, 5) fused column slice + uniform sampling without replacement, then unique + relabel; the frontier is
the next hop's seeds.  One STEP = one pass over the configuration's 1,000 minibatches on every GPU, handed to the
batched sampler `--group` minibatches per call.  The graph is replicated on every GPU and every GPU has its own 1,000
minibatches (weak scaling; minibatch b of the 1,000 x N goes to rank b mod N and its random stream is keyed by b, so
results do not depend on N); NCCL only reduces the run statistics.

Prints ONE JSON line (rank 0):
  value       timed with the seeds resident in HBM and per-kernel event timing off: exactly K steps between
              barrier + synchronize, repeated until the timed work adds up to >= 0.5 s; the median repeat is
              reported (`timing` carries min / median / max and the total);
  e2e         the same steps through the public operator (ops.sage_sample_batches -> C ABI) with the seeds copied
              from pinned host memory every call and the sizes of every hop read back on the host;
  e2e_dropin  the reference's own super-batch Python loop (its registered TorchScript names) on lib/libgs.so, and
              e2e_dropin_per_batch its per-minibatch Graph loop: what a user of the reference gets by swapping the library;
  roofline    per-kernel CUDA-event times from a separate untimed step; algorithmic bytes over the measured HBM peak;
  secondary   short legs of the other configurations (2-hop small graph, layer-wise, random walk, adaptive).
`--impl reference` times the reference's own implementation of the same steps: its CUDA library compiled unmodified
for sm_100 (oracle/_ref/libgs_ref.so) if it is present, because the reference has no CPU path; otherwise the CPU
restatement on the host cores.
"""
import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FANOUTS = [15, 10, 5]
BATCH = 1024
NUM_NODES = 2_450_000
NUM_EDGES = 123_700_000
MAX_DEGREE = 17_000
TRAIN_FRACTION = 0.08
GRAPH_SEED = 0x5EED + 2
RUN_SEED = 2024
METRIC = "sampled_edges_per_second"
UNIT = "edges/s"


# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) divided by algorithmic bytes, from one ncu capture per
# kernel on hop 3 of a 64-minibatch call of this workload (profiles/k_*_sage3hop_group64.md).  Traffic grows in
# proportion to the units a launch processes, so a full launch's traffic is this ratio times its algorithmic bytes.
TRAFFIC_OVER_ALGORITHMIC = {"sample_uniform": 4.2, "table_insert": 4.1, "first_compact": 3.2, "relabel": 1.04,
                            # partitioned form (profiles/k_part_*_sage3hop_group64.md, k_rank_emit_sage3hop_group64.md)
                            "partition_count": 1.04, "partition_scatter": 0.81, "bucket_resolve": 0.88,
                            "first_bits": 1.0}
# the same with direct-address tables (profiles/k_direct_insert_sage3hop_group64.md)
TRAFFIC_OVER_ALGORITHMIC_DIRECT = {"sample_uniform": 4.2, "table_insert": 9.1}


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batches-per-step", type=int, default=1000,
                    help="minibatches every GPU processes per step (the configuration has 1,000)")
    ap.add_argument("--relabel-path", default=None, choices=["auto", "hash", "direct", "partition"],
                    help="table form of unique + relabel (default: the library's automatic choice)")
    ap.add_argument("--lanes", type=int, default=3,
                    help="CUDA streams (each with its own library context and output arena) that take the calls of a "
                         "step in turn; with --host-waits every lane is a host thread")
    ap.add_argument("--host-waits", action="store_true",
                    help="wait on the host for the exact sizes after every hop (lanes then are host threads) instead of "
                         "queuing whole steps sized by hints from a first pass")
    ap.add_argument("--spin-wait", action="store_true",
                    help="with several lanes: let waiting lanes spin (cudaStreamSynchronize) instead of sleeping on an event")
    ap.add_argument("--min-timed-seconds", type=float, default=0.5,
                    help="the timed region is repeated until this much timed work exists (at least 3 repeats)")
    ap.add_argument("--no-dropin", action="store_true", help="skip the TorchScript drop-in legs")
    ap.add_argument("--dropin-steps", type=int, default=2)
    ap.add_argument("--dropin-batches", type=int, default=300)
    ap.add_argument("--secondary", dest="secondary", action="store_true", default=True,
                    help="after the headline, short legs of the other configurations (one GPU only)")
    ap.add_argument("--no-secondary", dest="secondary", action="store_false")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--nodes", type=int, default=NUM_NODES, help="override the graph size (debugging only)")
    ap.add_argument("--edges", type=int, default=NUM_EDGES)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--workload", default="sage", choices=["sage", "walk", "kernels", "ladies", "adaptive", "access", "atomics"],
                    help="sage = the headline (the products-scale configuration); walk = uniform random walk (papers-scale "
                         "configuration); ladies = layer-wise importance sampling (1 M nodes / 50 M weighted edges); adaptive = "
                         "SDDMM score -> per-column softmax -> weighted sampling on the products-scale graph; both of the "
                         "latter run the same TorchScript call sequence on our library or, with --impl reference, on the "
                         "reference's")
    ap.add_argument("--walkers", type=int, default=10_000_000)
    ap.add_argument("--walk-length", type=int, default=80)
    ap.add_argument("--walk-nodes", type=int, default=111_000_000)
    ap.add_argument("--walk-edges", type=int, default=1_600_000_000)
    ap.add_argument("--group", type=int, default=500,
                    help="minibatches handed to one call of the batched sampler")
    return ap.parse_args()


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML while a region is timed."""

    def __init__(self, index, period=0.05, enabled=True):
        super().__init__(daemon=True)
        self.index, self.period = index, period
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop_evt = threading.Event()
        self.ok = False
        if not enabled:  # only rank 0 polls NVML: concurrent polling from every rank slows the launch threads
            self.nv = None
            return
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
            self.ok = True
        except Exception:
            self.nv = None

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._stop_evt.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop_evt.wait(self.period)

    def stop(self):
        self._stop_evt.set()
        if self.is_alive():
            self.join(timeout=2)
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


def physical_gpu_index(local_index):
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_index])
        except Exception:
            return local_index
    return local_index


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def graph_info(indptr, indices, gen_seconds):
    deg = indptr[1:] - indptr[:-1]
    return {"nodes": int(indptr.numel() - 1), "edges": int(indices.numel()), "max_degree": int(deg.max().item())}, \
        round(gen_seconds, 2)


def make_inputs(args, device, world, rank):
    """The products-scale graph (replicated) and this rank's share of the configuration's minibatches: every rank
    processes BATCHES_PER_STEP minibatches per step (weak scaling), dealt round-robin from world x that many, and
    carries their GLOBAL numbers, which key the random streams."""
    import torch
    from graph_sampling_b200.synthetic import rmat_csc, seed_batches
    from graph_sampling_b200.sharding import shard_batches, shard_batch_ids
    t0 = time.time()
    indptr, indices = rmat_csc(args.nodes, args.edges, seed=GRAPH_SEED, symmetric=True, max_degree=MAX_DEGREE,
                               device=device)
    torch.cuda.synchronize()
    torch.cuda.empty_cache()  # the generator's temporaries are several GB; keep only the graph resident
    info, gen_s = graph_info(indptr, indices, time.time() - t0)
    total = args.batches_per_step * world
    allb = seed_batches(args.nodes, BATCH, total, seed=GRAPH_SEED + 1, train_fraction=TRAIN_FRACTION, device="cpu")
    return indptr, indices, shard_batches(allb, rank, world), shard_batch_ids(total, rank, world), info, gen_s


def workload_config(args, info):
    """The part of `config` both arms print identically."""
    return {"workload": "products-scale GraphSAGE 3-hop uniform sampling, fanouts [15,10,5], 1024 seeds/batch, relabel "
                        "per hop (the products-scale configuration); one step = one pass over the configuration's "
                        f"{args.batches_per_step} minibatches per GPU, handed to the sampler {args.group} at a time",
            "graph": info, "batch": BATCH, "fanouts": FANOUTS, "batches_per_step": args.batches_per_step,
            "group": args.group,
            "l2": "inputs larger than L2: 1 GB of indices gathered at random, no flush"}


def sage_batch_api(graph, seeds, fused_name, relabel_name):
    """The reference's per-batch loop (examples/graphsage/unbatching_training.py:19-28)."""
    fused = getattr(graph, fused_name)
    edges = 0
    shapes = []
    for k in FANOUTS:
        sub = fused(seeds, k, False)
        frontier, n_row, n_col, indptr, indices, e_ids, fmt = getattr(sub, relabel_name)()
        shapes.append((int(seeds.numel()), int(indices.numel()), int(n_row)))
        edges += int(indices.numel())
        seeds = frontier
    return edges, shapes


def superbatch_torchscript(torch, G, seeds, ptr):
    """The reference's own super-batch loop (examples/graphsage/batching.py:56-90) spelled with the registered
    TorchScript names: fused sampling over the seeds of all minibatches, per-batch edge offsets from the sampled
    CSC, gs_ops.BatchCSRRelabel.  Runs unchanged on the reference's library and on lib/libgs.so."""
    edges, shapes = 0, []
    for k in FANOUTS:
        sub = G._CAPI_FusedColumnwiseSlicingSampling(seeds, k, False)
        sub_indptr, sub_indices, _ = sub._CAPI_GetCSC()
        indices_ptr = sub_indptr[ptr]
        uniq, uniq_ptr, rel, _ = torch.ops.gs_ops._CAPI_BatchCSRRelabel(seeds, ptr, sub_indices, indices_ptr)
        shapes.append((int(seeds.numel()), int(sub_indices.numel()), int(uniq.numel())))
        edges += int(sub_indices.numel())
        seeds, ptr = uniq, uniq_ptr
    return edges, shapes


class Stepper:
    """One step = one pass over this rank's minibatches, `group` of them per call of `call(seeds_2d, first, step, lane)`
    (first = index of the group's first minibatch, step = number of the pass).  The source array may live on the
    device or in pinned host memory; a host source is copied group by group inside the step.

    lanes > 1: the groups of a step are dealt to that many host threads, each with its own CUDA stream (and, in the
    caller's `call`, its own library context and output arena), so that the host waits of one call overlap the device
    work of another.  Every lane stream starts a step after the work already queued on the current stream and the
    current stream continues after all lanes, so CUDA events recorded on the current stream bracket the step."""

    def __init__(self, torch, call, source, group, device, lanes=1, queued=None):
        self.torch, self.call, self.source, self.group, self.device = torch, call, source, group, device
        self.step_no = 0
        self.shapes = []
        self.keep_shapes = False
        self.lanes = max(1, int(lanes))
        self.streams, self.pool = [], None
        # queued = (call_queued, finish): the calls of a step are only QUEUED, by this one host thread, on `lanes`
        # streams in turn (call_queued(seeds_2d, first, step, lane) returns device-side counts), and finish(list of
        # those, step) waits once at the end of the step and returns (edges, shapes)
        self.queued = queued
        if self.lanes > 1 or queued is not None:
            self.streams = [torch.cuda.Stream(device=device) for _ in range(self.lanes)]
        if self.lanes > 1 and queued is None:
            from concurrent.futures import ThreadPoolExecutor
            self.pool = ThreadPoolExecutor(max_workers=self.lanes)

    def _run_lane(self, lane, firsts):
        torch = self.torch
        edges, shapes_out = 0, []
        torch.cuda.set_device(self.device)          # the current device is per thread
        stream = self.streams[lane] if self.streams else torch.cuda.current_stream()
        with torch.cuda.stream(stream):
            for first in firsts:
                sb = self.source[first:first + self.group]
                if not sb.is_cuda:
                    sb = sb.to(self.device, non_blocking=True)
                e, shapes = self.call(sb, first, self.step_no, lane)
                edges += e
                shapes_out.append(shapes)
        return edges, shapes_out

    def _step_queued(self, firsts):
        torch = self.torch
        call_queued, finish = self.queued
        main = torch.cuda.current_stream()
        for st in self.streams:
            st.wait_stream(main)
        pending = []
        for i, first in enumerate(firsts):
            lane = i % self.lanes
            with torch.cuda.stream(self.streams[lane]):
                sb = self.source[first:first + self.group]
                if not sb.is_cuda:
                    sb = sb.to(self.device, non_blocking=True)
                pending.append(call_queued(sb, first, self.step_no, lane))
        for st in self.streams:
            main.wait_stream(st)
        return finish(pending, self.step_no)

    def step(self):
        torch = self.torch
        firsts = list(range(0, self.source.shape[0], self.group))
        if self.queued is not None:
            edges, shapes = self._step_queued(firsts)
        elif self.lanes == 1:
            edges, shapes = self._run_lane(0, firsts)
        else:
            main = torch.cuda.current_stream()
            for st in self.streams:
                st.wait_stream(main)
            futures = [self.pool.submit(self._run_lane, lane, firsts[lane::self.lanes]) for lane in range(self.lanes)]
            results = [f.result() for f in futures]
            for st in self.streams:
                main.wait_stream(st)
            edges = sum(r[0] for r in results)
            shapes = [sh for r in results for sh in r[1]]
        if self.keep_shapes:
            self.shapes.extend(shapes)
        self.step_no += 1
        return edges


def timed_steps(torch, stepper, warmup, steps, barrier, reduce_max, min_seconds=0.5, min_repeats=3, max_repeats=25):
    """`warmup` untimed steps, then the timed region — exactly `steps` steps between barrier + synchronize on both
    sides, CUDA events on the launching stream — repeated until at least `min_seconds` of timed work and
    `min_repeats` repeats exist.  Every repeat's time is the max over ranks.  Returns (per-repeat seconds, edges of one
    repeat on this rank); the caller reports the median repeat."""
    for _ in range(warmup):
        stepper.step()
    seconds = []
    edges = 0
    while len(seconds) < max_repeats and (len(seconds) < min_repeats or sum(seconds) < min_seconds):
        torch.cuda.synchronize()
        barrier()
        torch.cuda.synchronize()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        edges = 0
        for _ in range(steps):
            edges += stepper.step()
        ev1.record()
        torch.cuda.synchronize()
        barrier()
        seconds.append(reduce_max(ev0.elapsed_time(ev1) / 1e3))
    return seconds, edges


def median(xs):
    s = sorted(xs)
    return s[len(s) // 2] if len(s) % 2 else 0.5 * (s[len(s) // 2 - 1] + s[len(s) // 2])


def cpu_baseline(indptr, indices, batches, limit_s=10.0, min_s=2.0):
    """Times the CPU restatement of the same batch loop on all host cores, on a bounded sample: whole minibatches
    for at least `min_s` and at most `limit_s` seconds, whatever --steps says."""
    from oracle import build as obuild
    obuild.build()
    from oracle import oracle as o
    ip, ix = indptr.cpu().numpy(), indices.cpu().numpy()
    o.sage_batch(ip, ix, batches[0].numpy(), FANOUTS, seed=1)  # warm
    t0, edges, n = time.time(), 0, 0
    while (time.time() - t0) < min_s or (n < len(batches) and (time.time() - t0) < limit_s):
        edges += o.sage_batch(ip, ix, batches[n % len(batches)].numpy(), FANOUTS, seed=n, batch_id=n)
        n += 1
    dt = time.time() - t0
    return {"value": edges / dt, "unit": UNIT, "cores": o.num_threads(), "kind": "port",
            "sample": f"{n} minibatches of {BATCH} seeds of the same workload ({dt:.1f} s)"}


def run_ours(args):
    import torch
    rank, world, local = dist_env()
    dist = None
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)
    barrier = (lambda: dist.barrier()) if world > 1 else (lambda: None)

    def reduce_max(x):
        if world == 1:
            return float(x)
        t = torch.tensor([x], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def reduce_sum(x):
        if world == 1:
            return int(x)
        t = torch.tensor([float(x)], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return int(round(t.item()))

    from graph_sampling_b200 import ops
    indptr, indices, batches, batch_ids, info, gen_s = make_inputs(args, device, world, rank)
    lanes = max(1, args.lanes)
    # one library context (scratch, counters) and one output arena per lane: calls of different lanes overlap
    ctxs = [ops.default_context(device)] + [ops.Context(device) for _ in range(lanes - 1)]
    ctx = ctxs[0]
    for c in ctxs:
        if args.relabel_path:
            c.set_option("relabel_path", {"auto": 0, "hash": 1, "direct": 2, "partition": 3}[args.relabel_path])
        if args.host_waits and lanes > 1 and not args.spin_wait:
            c.set_option("blocking_wait", 1)    # a lane that waits for its hop sleeps; the other lanes keep the GPU fed
    group = args.group
    ids_dev = batch_ids.to(device)
    ptr_cache = {}
    arenas = [ops.OutputArena() for _ in range(lanes)]

    def call_batched(sb, first, step_no, lane=0):
        """`group` minibatches through the batched sampler: per hop one call of the C ABI (gsb_sage_hop: fused slice +
        sample, then unique + relabel of every minibatch), one host wait per hop for the exact sizes (queuing all hops
        on upper bounds was measured slower: the bounds overshoot 3.5x)."""
        g, s0 = sb.shape
        ptr = ptr_cache.get(g)
        if ptr is None:
            ptr = ptr_cache[g] = torch.arange(g + 1, dtype=torch.int64, device=device) * s0
        hops = ops.sage_sample_batches(indptr, indices, sb.reshape(-1), ptr, FANOUTS, replace=False,
                                       seed=RUN_SEED + 8 * step_no, arena=arenas[lane], ctx=ctxs[lane],
                                       batch_ids=ids_dev[first:first + g], seeds_distinct=True)
        shapes = [(int(h["seeds"].numel()), int(h["indices"].numel()), int(h["frontier"].numel())) for h in hops]
        return sum(e for _, e, _ in shapes), shapes

    # ---- size hints: one pass with host waits records the sizes of every call of a step; the timed steps then queue
    # their calls without waiting, sized by these figures plus a margin (what a training loop has from its previous
    # epoch).  A call that outgrows its hint reports it and is repeated the slow way.
    dev_batches = batches.to(device)
    for g in sorted({min(group, batches.shape[0]), batches.shape[0] % group} - {0}):   # offset arrays, made once
        ptr_cache[g] = torch.arange(g + 1, dtype=torch.int64, device=device) * BATCH
    sized = Stepper(torch, call_batched, dev_batches, group, device, 1)
    sized.keep_shapes = True
    sized.step()  # also sizes scratch, the output arenas and the tables before anything is timed
    firsts = list(range(0, batches.shape[0], group))
    hints = {first: [(int(s_ * 1.03) + 1024, int(e_ * 1.03) + 1024) for s_, e_, _ in sh]
             for first, sh in zip(firsts, sized.shapes)}
    overflow = {"calls": 0}

    def call_queued(sb, first, step_no, lane=0):
        g, s0 = sb.shape
        hops = ops.sage_sample_batches(indptr, indices, sb.reshape(-1), ptr_cache[g], FANOUTS, replace=False,
                                       seed=RUN_SEED + 8 * step_no, arena=arenas[lane], ctx=ctxs[lane], sync=False,
                                       batch_ids=ids_dev[first:first + g], seeds_distinct=True, size_hints=hints[first])
        return torch.stack([h["counts"] for h in hops])          # [hops, 3] on the device: seeds, edges, frontier

    def finish_step(pending, step_no):
        counts = torch.stack(pending).cpu()                       # the one host wait of the step
        for c in ctxs:
            try:
                c.check_device()
            except ops.GsbError:                                  # a hint was too small: say so (the figures would be wrong)
                overflow["calls"] += 1
                raise
        shapes = [[tuple(int(x) for x in hop) for hop in call] for call in counts]
        return int(counts[:, :, 1].sum()), shapes

    queued = None if args.host_waits else (call_queued, finish_step)
    # ---- value: seeds resident in HBM, per-kernel event timing OFF -----------------------------------------
    stepper = Stepper(torch, call_batched, dev_batches, group, device, lanes, queued)
    stepper.step()
    sampler = ClockSampler(physical_gpu_index(local), enabled=(rank == 0))
    sampler.start()
    launches0 = sum(c.launch_count() for c in ctxs)
    steps_before = stepper.step_no
    seconds, edges = timed_steps(torch, stepper, args.warmup, args.steps, barrier, reduce_max,
                                 min_seconds=args.min_timed_seconds)
    launches = (sum(c.launch_count() for c in ctxs) - launches0) * args.steps // max(1, stepper.step_no - steps_before)
    clocks = sampler.stop()
    edges_all = reduce_sum(edges)
    sec_med = median(seconds)

    # ---- e2e: the same steps with the seeds in pinned host memory; sizes of every hop read back on the host -----
    pinned = batches.pin_memory()
    e2e_stepper = Stepper(torch, call_batched, pinned, group, device, lanes, queued)
    e2e_seconds, e2e_edges = timed_steps(torch, e2e_stepper, min(args.warmup, 2), args.steps, barrier, reduce_max,
                                         min_seconds=args.min_timed_seconds)
    e2e_edges_all = reduce_sum(e2e_edges)
    e2e_med = median(e2e_seconds)
    calls_per_step = (batches.shape[0] + group - 1) // group

    # ---- per-kernel device time: a separate, untimed pass of one step with event timing on ----------------------
    prof_stepper = Stepper(torch, call_batched, dev_batches, group, device)      # one lane: kernels one after another
    prof_stepper.step()                                                          # untimed: buffers of this lane grow here
    torch.cuda.synchronize()
    prof_stepper.keep_shapes = True
    ctx.profile_reset()
    ctx.profile_enable(True)
    prof_stepper.step()
    torch.cuda.synchronize()
    ctx.profile_enable(False)
    prof = ctx.profile_read()
    shapes = prof_stepper.shapes

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- drop-in: the reference's own call sequence on lib/libgs.so (one GPU, rank 0) ---------------------------
    dropin = dropin_torchscript(torch, args, device, indptr, indices, pinned) if not args.no_dropin else None

    # ---- roofline of the dominant kernel (largest share of device time in the profiled step) --------------------
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        peak, peak_src = float(json.load(open(peaks_path))["hbm_gbs"]), "measured"
    else:
        peak, peak_src = 6650.0, "fallback"
    # Algorithmic bytes per launch of each hot kernel, from the shapes of the profiled calls: (S, E, U) per hop.
    # sample: 32 B per seed column (seed id, indptr pair, output offset) + 24 B per sampled edge (8 read, 16 written);
    # unique + relabel, hash-region / direct-table forms: three passes over N = S + E items: insert reads 8 N;
    # first-occurrence compaction reads 8 N and writes 8 U; relabel reads 8 E and writes 8 E (table traffic is overhead,
    # not counted).  Partitioned form: count reads 8 N; scatter reads 8 N and writes 8 N; the per-bucket resolve reads
    # 8 N and writes 4 N; the bit pass reads 4 N; the emit pass reads 4 N and the 8 U ids of the first occurrences and
    # writes 8 U + 8 E.
    hop_shapes = [h for call in shapes for h in call]
    n_launch = max(1, len(hop_shapes))
    alg = {
        "sample_uniform": sum(32 * s_ + 8 + 24 * e_ for s_, e_, _ in hop_shapes) / n_launch,
        "table_insert": sum(8 * (s_ + e_) for s_, e_, _ in hop_shapes) / n_launch,
        "first_compact": sum(8 * (s_ + e_) + 8 * u_ for s_, e_, u_ in hop_shapes) / n_launch,
        "relabel": sum(16 * e_ for s_, e_, _ in hop_shapes) / n_launch,
        "partition_count": sum(8 * (s_ + e_) for s_, e_, _ in hop_shapes) / n_launch,
        "partition_scatter": sum(16 * (s_ + e_) for s_, e_, _ in hop_shapes) / n_launch,
        "bucket_resolve": sum(12 * (s_ + e_) for s_, e_, _ in hop_shapes) / n_launch,
        "first_bits": sum(4 * (s_ + e_) for s_, e_, _ in hop_shapes) / n_launch,
        "rank_emit": sum(4 * (s_ + e_) + 16 * u_ + 8 * e_ for s_, e_, u_ in hop_shapes) / n_launch,
    }
    # which form of unique + relabel ran is read off the kernels that were launched
    launched = {name for name, (ms, n) in prof.items() if n}
    form = "partition" if "bucket_resolve" in launched else "hash" if "table_clear" in launched else "direct"
    direct = form == "direct"
    form_text = {"partition": "shared-memory tables per bucket of items (partitioned form)",
                 "hash": "hash-table regions in global memory", "direct": "direct-address tables"}[form]
    kernel_names = {"sample_uniform": "k_sample_uniform_tpc (fused count + scan + uniform sample)",
                    "partition_count": "k_part_count (items per bucket)",
                    "partition_scatter": "k_part_scatter (items grouped by bucket)",
                    "bucket_resolve": "k_part_resolve (first position per id in a shared-memory table per bucket)",
                    "first_bits": "k_first_bits (bit vector of first occurrences)",
                    "rank_emit": "k_rank_emit (frontier and relabelled ids from the rank bit vector)",
                    "table_insert": "k_direct_insert (atomicMin into per-minibatch direct-address tables)" if direct
                    else "k_batch_insert (position-min hash insert)",
                    "first_compact": "k_direct_compact (first-occurrence test + scan + compaction)" if direct
                    else "k_direct_compact<HASH> (first-occurrence test on hash regions + scan + compaction)",
                    "relabel": "k_direct_fixup (rank look-up of repeated ids)"}
    total_ms = sum(v[0] for v in prof.values()) or 1.0
    per_kernel = {}
    for name, (ms, n) in prof.items():
        entry = {"ms": round(ms, 3), "launches": n, "share": round(ms / total_ms, 4)}
        if name in alg and n:
            avg_s = ms / 1e3 / n
            entry["avg_launch_us"] = round(avg_s * 1e6, 2)
            entry["bytes_per_launch"] = round(alg[name])
            entry["achieved_gbs"] = round(alg[name] / avg_s / 1e9, 2)
            entry["frac"] = round(alg[name] / avg_s / 1e9 / peak, 5)
            ratio = (TRAFFIC_OVER_ALGORITHMIC_DIRECT if direct else TRAFFIC_OVER_ALGORITHMIC).get(name)
            if ratio is not None:
                entry["traffic"] = round(alg[name] * ratio)
        per_kernel[name] = entry
    top = max((k for k in per_kernel if k in alg), key=lambda k: per_kernel[k]["ms"], default=None)
    if top is not None:
        t = per_kernel[top]
        roofline = {"bound": "hbm", "kernel": kernel_names[top], "achieved": t["achieved_gbs"], "peak": peak,
                    "peak_source": peak_src, "unit": "GB/s", "frac": t["frac"], "traffic": t.get("traffic"),
                    "traffic_source": "ncu capture of one launch on a 64-minibatch call, scaled by algorithmic bytes",
                    "bytes_per_launch": t["bytes_per_launch"], "avg_launch_us": t["avg_launch_us"],
                    "share_of_device_time": t["share"],
                    "measured": "CUDA events around every launch of one untimed step", "kernels": per_kernel}
    else:
        roofline = {"bound": "hbm", "kernel": None, "achieved": None, "peak": peak, "peak_source": peak_src,
                    "unit": "GB/s", "frac": None, "traffic": None, "kernels": per_kernel}
    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        cpu = cpu_baseline(indptr, indices, batches)
    line = {
        "metric": METRIC, "value": edges_all / sec_med, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": sec_med / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int64", "data": "synthetic",
        "config": workload_config(args, info),
        "arm": {"path": "batched sampler through the C ABI (gsb_sage_hop per hop: fused slice+sample, then unique + "
                        "relabel of every minibatch with %s)" % form_text,
                "parallelism": f"replicated graph, dp{world}; minibatch b of {args.batches_per_step * world} on rank "
                               "b mod N, random streams keyed by the global minibatch number",
                "graph_gen_seconds": gen_s, "relabel_path": form,
                "lanes": (f"{lanes} host thread(s), each with its own CUDA stream, library context and output arena, take "
                          "alternate calls of a step; one host wait per hop") if args.host_waits else
                         (f"one host thread queues the calls of a step on {lanes} CUDA stream(s) in turn (own library "
                          "context and output arena each), buffers sized by the first pass's sizes + 3 %, one host wait "
                          "per step"),
                "hint_overflows": overflow["calls"]},
        "edges_per_step": edges_all / args.steps / world,
        "timing": {"repeats": len(seconds), "timed_region_s": round(sum(seconds), 4),
                   "ms_per_step_min_median_max": [round(min(seconds) / args.steps * 1e3, 4),
                                                  round(sec_med / args.steps * 1e3, 4),
                                                  round(max(seconds) / args.steps * 1e3, 4)],
                   "reported": "median repeat; every repeat times exactly `steps` steps, max over ranks"},
        "e2e": {"value": e2e_edges_all / e2e_med, "unit": UNIT,
                "h2d_bytes_per_step": batches.shape[0] * BATCH * 8,
                "d2h_bytes_per_step": calls_per_step * len(FANOUTS) * (32 if args.host_waits else 24) +
                (0 if args.host_waits else lanes * 16),
                "ms_per_step": e2e_med / args.steps * 1e3, "repeats": len(e2e_seconds),
                "path": "ops.sage_sample_batches -> C ABI, seeds from pinned host memory every call, sizes of every hop "
                        "and the status read back; the sampled blocks stay in HBM (as in the reference's API)"},
        "gpu_launches": int(launches), "lanes": lanes,
        "clocks": clocks,
        "roofline": roofline,
    }
    if dropin is not None:
        line["e2e_dropin"] = dropin["super_batch"]
        line["e2e_dropin_per_batch"] = dropin["per_batch"]
    if cpu is not None:
        line["cpu_baseline"] = cpu
    if world == 1 and args.secondary:
        del dev_batches, pinned
        line["secondary"] = secondary_workloads(args, "ours", device, indptr, indices)
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def dropin_torchscript(torch, args, device, indptr, indices, pinned, lib_path=None):
    """The reference-facing TorchScript face timed end to end with the reference's own Python loops, seeds from pinned
    host memory: (1) its super-batch loop (fused sampling, GetCSC offsets, gs_ops.BatchCSRRelabel) on whole steps,
    (2) its per-minibatch Graph loop on a bounded sample.  `lib_path` None = lib/libgs.so (this repository's library)."""
    if lib_path is None:
        from graph_sampling_b200 import build as gsb_build
        lib_path = gsb_build.build_glue()
    torch.classes.load_library(lib_path)
    G = torch.classes.gs_classes.Graph(False)
    G._CAPI_LoadCSC(indptr, indices)
    ptr_cache = {}

    def call(sb, first, step_no, lane=0):
        g, s0 = sb.shape
        ptr = ptr_cache.get(g)
        if ptr is None:
            ptr = ptr_cache[g] = torch.arange(g + 1, dtype=torch.int64, device=device) * s0
        return superbatch_torchscript(torch, G, sb.reshape(-1), ptr)

    out = {}
    best = None
    for group in sorted({args.group, 250, 125}):
        st = Stepper(torch, call, pinned, group, device)
        steps = max(1, min(args.steps, args.dropin_steps))
        seconds, edges = timed_steps(torch, st, 1, steps, lambda: None, float, min_seconds=0.0, min_repeats=1,
                                     max_repeats=1)
        r = {"value": edges / seconds[0], "unit": UNIT, "group": group, "steps": steps,
             "ms_per_step": seconds[0] / steps * 1e3}
        if best is None or r["value"] > best["value"]:
            best = r
    best["path"] = ("TorchScript classes: _CAPI_FusedColumnwiseSlicingSampling -> _CAPI_GetCSC -> "
                    "gs_ops._CAPI_BatchCSRRelabel per hop (examples/graphsage/batching.py:56-90)")
    out["super_batch"] = best
    n = min(pinned.shape[0], args.dropin_batches)
    for b in range(5):
        sage_batch_api(G, pinned[b].to(device, non_blocking=True), "_CAPI_FusedColumnwiseSlicingSampling", "_CAPI_Relabel")
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    edges = 0
    for b in range(n):
        e, _ = sage_batch_api(G, pinned[b].to(device, non_blocking=True), "_CAPI_FusedColumnwiseSlicingSampling",
                              "_CAPI_Relabel")
        edges += e
    ev1.record()
    torch.cuda.synchronize()
    sec = ev0.elapsed_time(ev1) / 1e3
    out["per_batch"] = {"value": edges / sec, "unit": UNIT, "minibatches": n, "ms_per_minibatch": sec / n * 1e3,
                        "path": "TorchScript Graph per minibatch and hop: _CAPI_FusedColumnwiseSlicingSampling, "
                                "_CAPI_Relabel (examples/graphsage/unbatching_training.py:19-28)"}
    return out


def run_reference(args):
    """Reference arm.  The reference implements this path in CUDA only (every dispatcher aborts off-GPU), so its own
    implementation — its sources compiled unmodified for sm_100 — is timed on the GPU through its TorchScript classes
    with its own loops, on the same steps; if the compiled library is absent the CPU restatement is timed on the host
    cores instead."""
    rank, world, local = dist_env()
    if rank != 0:
        return
    import torch
    lib = os.path.join(ROOT, "oracle", "_ref", "libgs_ref.so")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    indptr, indices, batches, _, info, gen_s = make_inputs(args, device, 1, 0)
    base = {"metric": METRIC, "unit": UNIT, "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int64", "data": "synthetic",
            "impl": "reference", "config": workload_config(args, info)}
    if os.path.exists(lib):
        pinned = batches.pin_memory()
        sampler = ClockSampler(physical_gpu_index(local))
        sampler.start()
        torch.classes.load_library(lib)
        G = torch.classes.gs_classes.Graph(False)
        G._CAPI_LoadCSC(indptr, indices)
        ptr_cache = {}

        def call(sb, first, step_no, lane=0):
            g, s0 = sb.shape
            ptr = ptr_cache.get(g)
            if ptr is None:
                ptr = ptr_cache[g] = torch.arange(g + 1, dtype=torch.int64, device=device) * s0
            return superbatch_torchscript(torch, G, sb.reshape(-1), ptr)

        # its super-batch loop at this run's group size and at the 256-ish size its examples use: one trial step
        # each, the faster one is measured in full
        trial = {}
        for group in sorted({args.group, 250, 125}):
            st = Stepper(torch, call, pinned, group, device)
            sec, e = timed_steps(torch, st, 1, 1, lambda: None, float, min_seconds=0.0, min_repeats=1, max_repeats=1)
            trial[group] = e / sec[0]
        group = max(trial, key=trial.get)
        st = Stepper(torch, call, pinned, group, device)
        seconds, edges = timed_steps(torch, st, args.warmup, args.steps, lambda: None, float, min_seconds=0.5,
                                     min_repeats=1, max_repeats=3)
        sec_med = median(seconds)
        batched = edges / sec_med
        # its per-minibatch Graph loop on a bounded sample
        n = min(pinned.shape[0], 500)
        for b in range(5):
            sage_batch_api(G, pinned[b].to(device, non_blocking=True), "_CAPI_FusedColumnwiseSlicingSampling", "_CAPI_Relabel")
        torch.cuda.synchronize()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        pb_edges = 0
        for b in range(n):
            e, _ = sage_batch_api(G, pinned[b].to(device, non_blocking=True), "_CAPI_FusedColumnwiseSlicingSampling",
                                  "_CAPI_Relabel")
            pb_edges += e
        ev1.record()
        torch.cuda.synchronize()
        pb_sec = ev0.elapsed_time(ev1) / 1e3
        per_batch = pb_edges / pb_sec
        clocks = sampler.stop()
        if batched >= per_batch:
            v, ms_step = batched, sec_med / args.steps * 1e3
        else:
            v, ms_step = per_batch, pb_sec / n * args.batches_per_step * 1e3
        base["arm"] = {"reference_paths": {"per_batch_graph_api_edges_per_s": per_batch,
                                           "super_batch_edges_per_s": batched, "super_batch_group": group,
                                           "super_batch_trials_edges_per_s": trial,
                                           "reported": "super-batch" if batched >= per_batch else "per-batch"},
                       "graph_gen_seconds": gen_s, "repeats": len(seconds)}
        base.update({"value": v, "ms_per_step": ms_step, "clocks": clocks,
                     "cpu_baseline": {"value": v, "unit": UNIT, "cores": 0, "kind": "reference",
                                      "sample": "the reference has no CPU path; this is its own CUDA library "
                                                "(unmodified sources compiled for sm_100) on the same GPU, "
                                                f"{args.steps} steps of {args.batches_per_step} minibatches"},
                     "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}})
        if args.secondary:
            del pinned
            base["secondary"] = secondary_workloads(args, "reference", device, indptr, indices)
    else:
        cpu = cpu_baseline(indptr, indices, batches, limit_s=60.0)
        base.update({"value": cpu["value"], "ms_per_step": None, "cpu_baseline": cpu,
                     "e2e": {"value": cpu["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}})
    print(json.dumps(base))


def measure_walk(torch, args, impl, device, rank=0, world=1, barrier=lambda: None, steps=3, warmup=1):
    """Uniform random walk (papers-scale configuration): one walker per distinct start node, walkers split into
    contiguous ranges over the ranks, int64 trace [walkers, length + 1].  A step is one full pass over this rank's
    walkers.  Returns this rank's figures (the caller reduces over ranks)."""
    from graph_sampling_b200.synthetic import rmat_csc, distinct_starts
    from graph_sampling_b200.sharding import shard_walkers
    from graph_sampling_b200 import validate
    t0 = time.time()
    indptr, indices = rmat_csc(args.walk_nodes, args.walk_edges, seed=GRAPH_SEED + 4, device=device, permute=True)
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    info = {"nodes": args.walk_nodes, "edges": int(indices.numel())}
    gen_s = round(time.time() - t0, 1)
    starts = distinct_starts(args.walk_nodes, args.walkers, seed=7, device=device)
    off, cnt = shard_walkers(args.walkers, rank, world)
    mine = starts[off:off + cnt].contiguous()
    L = args.walk_length
    if impl == "reference":
        torch.classes.load_library(os.path.join(ROOT, "oracle", "_ref", "libgs_ref.so"))
        G = torch.classes.gs_classes.Graph(False)
        G._CAPI_LoadCSC(indptr, indices)
        fn = lambda: G._CAPI_RandomWalk(mine, L)
    else:
        from graph_sampling_b200 import ops
        # layout 0 = the reference's own memory order, so both arms write the same layout
        fn = lambda: ops.fused_random_walk(mine, L, indices, indptr, layout=0, walker_offset=off, seed=RUN_SEED)
    for _ in range(warmup):
        out = fn()
    torch.cuda.synchronize()
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(steps):
        out = fn()
    ev1.record()
    torch.cuda.synchronize()
    seconds = ev0.elapsed_time(ev1) / 1e3
    check = validate.check_walk_trace(indptr, indices, out, cnt, L, step_major=True, sample=100_000)
    check["ok_start_nodes"] = bool(torch.equal(out.reshape(-1)[:cnt], mine))
    alive = float((out >= 0).float().mean().item()) if out.numel() < (1 << 31) else None
    del out
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    peak = float(json.load(open(peaks_path))["hbm_gbs"]) if os.path.exists(peaks_path) else 6650.0
    alg = (16 * cnt + 32 * cnt * L)  # per pass on this rank
    ach = alg * steps / seconds / 1e9
    return {"seconds": seconds, "units": cnt * L * steps, "steps": steps, "warmup": warmup, "graph": info,
            "graph_gen_seconds": gen_s, "fraction_of_trace_alive": alive, "checked": check,
            "checks_pass": validate.all_ok(check),
            "roofline": {"bound": "hbm", "kernel": "k_random_walk", "achieved": round(ach, 2), "peak": peak,
                         "unit": "GB/s", "frac": round(ach / peak, 5), "traffic": None}}


def run_walk(args):
    """`--workload walk`: prints its own JSON line (metric walker_steps_per_second)."""
    import torch
    rank, world, local = dist_env()
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)
    barrier = (lambda: dist.barrier()) if world > 1 else (lambda: None)
    from graph_sampling_b200.sharding import reduce_run_stats
    steps, warmup = max(1, min(args.steps, 5)), max(1, min(args.warmup, 2))
    args.walkers = min(args.walkers, args.walk_nodes)      # one walker per DISTINCT start node
    m = measure_walk(torch, args, args.impl, device, rank, world, barrier, steps, warmup)
    seconds_all, units_all = reduce_run_stats(m["seconds"], m["units"], device=device)
    if rank == 0:
        print(json.dumps({"metric": "walker_steps_per_second", "value": units_all / seconds_all, "unit": "steps/s",
                          "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": seconds_all / steps * 1e3,
                          "higher_is_better": True, "scaling": "strong", "dtype": "int64", "data": "synthetic",
                          "impl": args.impl,
                          "config": {"workload": "uniform random walk (papers-scale configuration)", "graph": m["graph"],
                                     "walkers": args.walkers, "length": args.walk_length,
                                     "layout": "step-major memory (the reference's own)",
                                     "fraction_of_trace_alive": m["fraction_of_trace_alive"]},
                          "checked": m["checked"], "roofline": m["roofline"]}))
    if world > 1:
        dist.destroy_process_group()


def _load_face(impl):
    """torch.classes.gs_classes.Graph and torch.ops.gs_ops of our TorchScript library or of the reference's."""
    import torch
    if impl == "reference":
        torch.classes.load_library(os.path.join(ROOT, "oracle", "_ref", "libgs_ref.so"))
    else:
        from graph_sampling_b200 import build as gsb_build
        torch.classes.load_library(gsb_build.build_glue())
    return torch.classes.gs_classes.Graph, torch.ops.gs_ops


_COO, _CSC, _CSR = 1, 2, 4


def ladies_batch(torch, gs_ops, P, seeds, fanouts):
    """examples/ladies/train_minibatch.py:43-59 spelled with the registered methods that gs.Matrix forwards to
    (python/gs/matrix_api/matrix.py:66-105): column slice, row probability = sum of squared weights, weighted list
    sampling, row slice, divide, normalise, frontier + relabel.  Returns the edges of the layer blocks."""
    edges = 0
    for fanout in fanouts:
        U = P._CAPI_Slicing(seeds, 0, _CSC, _COO, False)
        prob = U._CAPI_Sum(1, 2, _CSR)
        selected, _ = gs_ops._CAPI_ListSamplingWithProbs(U._CAPI_GetRows(), prob, fanout, False)
        nodes = torch.cat((seeds, selected)).unique()
        subU = U._CAPI_Slicing(nodes, 1, _CSR, _COO, False)
        subU = subU._CAPI_Divide(prob[nodes], 1, _COO)._CAPI_Normalize(0, _CSC)
        seeds = subU._CAPI_AllValidNode()
        subU._CAPI_Relabel()
        edges += int(subU._CAPI_GetNumEdges())
    return edges


def adaptive_batch(torch, gs_ops, A, X, seeds, fanouts):
    """Adaptive sampling hop by hop: column slice, edge score <x_src, x_dst> / 16 by SDDMM, per-column softmax,
    weighted sampling without replacement, frontier + relabel.  Returns the sampled edges."""
    edges = 0
    for fanout in fanouts:
        sub = A._CAPI_Slicing(seeds, 0, _CSC, _COO, False)
        score = torch.zeros(int(sub._CAPI_GetNumEdges()), 1, dtype=torch.float32, device=seeds.device)
        sub._CAPI_SDDMM("dot", X, X[seeds], score, 0, 2, _COO)
        sub._CAPI_SetData(torch.exp(score.squeeze(-1) / 16.0))
        p = sub._CAPI_Normalize(0, _CSC)._CAPI_GetData("default")
        sampled = sub._CAPI_SamplingWithProbs(0, p, fanout, False, _CSC, _CSC)
        seeds = sampled._CAPI_AllValidNode()
        sampled._CAPI_Relabel()
        edges += int(sampled._CAPI_GetNumEdges())
    return edges


PIPELINES = {
    "ladies": {"nodes": 1_000_000, "edges": 50_000_000, "batch": 512, "fanouts": [512, 512], "symmetric": False,
               "text": "layer-wise importance sampling: per layer column-slice 512 seeds, row probability = sum of squared "
                       "edge weights, 512 rows without replacement by that probability, row-slice, divide + normalise, "
                       "relabel; 2 layers; R-MAT 1 M nodes / 50 M edges, fp32 weights ~ U(0, 1]",
               "unit_text": "edges of the row-sliced layer blocks"},
    "adaptive": {"nodes": NUM_NODES, "edges": NUM_EDGES, "batch": 2048, "fanouts": [10, 10], "symmetric": True,
                 "text": "adaptive sampling on the products-scale graph, features fp32 [nodes x 256] ~ N(0, 1): per hop "
                         "column-slice, SDDMM score <x_src, x_dst> / 16, per-column softmax, weighted sampling without "
                         "replacement (fanout 10), relabel; 2 hops; 2 048 seeds per batch",
                 "unit_text": "sampled edges"},
}


def measure_pipeline(torch, workload, impl, device, steps, warmup, graph=None):
    """The two pipelines around weighted sampling, driven through the registered TorchScript methods, so that
    impl="reference" runs the very same Python loop on the reference's own CUDA library.  One GPU; a step is one
    minibatch; seeds come from pinned host memory inside the timed region.  `graph` = (indptr, indices) to reuse."""
    from graph_sampling_b200.synthetic import rmat_csc, seed_batches
    cfg = PIPELINES[workload]
    Graph, gs_ops = _load_face(impl)
    t0 = time.time()
    if graph is None:
        kw = {"symmetric": True, "max_degree": MAX_DEGREE} if cfg["symmetric"] else {}
        graph_seed = GRAPH_SEED if workload == "adaptive" else GRAPH_SEED + 3
        indptr, indices = rmat_csc(cfg["nodes"], cfg["edges"], seed=graph_seed, device=device, **kw)
        torch.cuda.synchronize()
        torch.cuda.empty_cache()
    else:
        indptr, indices = graph
    n = int(indptr.numel() - 1)
    info = {"nodes": n, "edges": int(indices.numel())}
    gen_s = round(time.time() - t0, 2)
    gen = torch.Generator(device=device)
    gen.manual_seed(GRAPH_SEED + 11)
    G = Graph(False)
    G._CAPI_LoadCSC(indptr, indices)
    X = None
    if workload == "ladies":
        w = 1.0 - torch.rand(indices.numel(), generator=gen, device=device)  # (0, 1]
        G._CAPI_SetData(w)
    else:
        X = torch.randn(n, 256, generator=gen, device=device)
    batches = seed_batches(n, cfg["batch"], steps + warmup, seed=GRAPH_SEED + 12, device="cpu").pin_memory()

    def fn(host_seeds):
        seeds = host_seeds.to(device, non_blocking=True)
        if workload == "ladies":
            return ladies_batch(torch, gs_ops, G, seeds, cfg["fanouts"])
        return adaptive_batch(torch, gs_ops, G, X, seeds, cfg["fanouts"])

    for b in range(warmup):
        fn(batches[b])
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    edges = 0
    ev0.record()
    for b in range(warmup, warmup + steps):
        edges += fn(batches[b])
    ev1.record()
    torch.cuda.synchronize()
    seconds = ev0.elapsed_time(ev1) / 1e3
    return {"value": edges / seconds, "unit": UNIT, "steps": steps, "warmup": warmup, "ms_per_step": seconds / steps * 1e3,
            "edges_per_step": edges / steps, "graph": info, "graph_gen_seconds": gen_s, "batch": cfg["batch"],
            "fanouts": cfg["fanouts"], "counted": cfg["unit_text"], "workload": cfg["text"]}


def run_pipeline(args):
    """`--workload ladies|adaptive`: prints its own JSON line."""
    rank, world, local = dist_env()
    if rank != 0:
        return
    import torch
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    steps, warmup = max(1, min(args.steps, 200)), max(3, min(args.warmup, 10))
    sampler = ClockSampler(physical_gpu_index(local))
    sampler.start()
    m = measure_pipeline(torch, args.workload, args.impl, device, steps, warmup)
    clocks = sampler.stop()
    print(json.dumps({"metric": METRIC, "value": m["value"], "unit": UNIT, "n_gpus": 1, "steps": steps,
                      "warmup": warmup, "ms_per_step": m["ms_per_step"], "higher_is_better": True,
                      "scaling": "weak", "vs_baseline": None, "dtype": "int64 ids, f32 weights", "data": "synthetic",
                      "impl": args.impl,
                      "config": {"workload": m["workload"], "graph": m["graph"], "batch": m["batch"],
                                 "fanouts": m["fanouts"], "counted": m["counted"],
                                 "face": "TorchScript classes (same call sequence for both arms)",
                                 "l2": "graph (and features) larger than L2, read at random"},
                      "edges_per_step": m["edges_per_step"], "clocks": clocks,
                      "e2e": {"value": m["value"], "unit": UNIT, "h2d_bytes_per_step": m["batch"] * 8,
                              "d2h_bytes_per_step": 8 * len(m["fanouts"])}}))


def measure_small_sage(torch, impl, device, group=125, steps=3):
    """The small GraphSAGE configuration: R-MAT 100,000 nodes / 2,000,000 directed edges, 1,000 minibatches of 1,024
    seeds drawn from all nodes, fanouts [10, 5], relabel per hop.  Ours: the batched sampler; reference: its own
    super-batch loop on its library.  A step is one pass over the 1,000 minibatches."""
    from graph_sampling_b200.synthetic import rmat_csc, seed_batches
    indptr, indices = rmat_csc(100_000, 2_000_000, seed=GRAPH_SEED - 1, device=device)
    batches = seed_batches(100_000, BATCH, 1000, seed=GRAPH_SEED + 20, device="cpu").pin_memory()
    fan = [10, 5]
    ptr_cache = {}

    def ptr_for(g, s0):
        if g not in ptr_cache:
            ptr_cache[g] = torch.arange(g + 1, dtype=torch.int64, device=device) * s0
        return ptr_cache[g]

    if impl == "reference":
        torch.classes.load_library(os.path.join(ROOT, "oracle", "_ref", "libgs_ref.so"))
        G = torch.classes.gs_classes.Graph(False)
        G._CAPI_LoadCSC(indptr, indices)

        def call(sb, first, step_no, lane=0):
            seeds, ptr = sb.reshape(-1), ptr_for(*sb.shape)
            edges = 0
            for k in fan:
                sub = G._CAPI_FusedColumnwiseSlicingSampling(seeds, k, False)
                sub_indptr, sub_indices, _ = sub._CAPI_GetCSC()
                seeds, ptr, _, _ = torch.ops.gs_ops._CAPI_BatchCSRRelabel(seeds, ptr, sub_indices, sub_indptr[ptr])
                edges += int(sub_indices.numel())
            return edges, None
    else:
        from graph_sampling_b200 import ops
        arena = ops.OutputArena()
        ids = torch.arange(1000, dtype=torch.int64, device=device)

        def call(sb, first, step_no, lane=0):
            hops = ops.sage_sample_batches(indptr, indices, sb.reshape(-1), ptr_for(*sb.shape), fan, seed=RUN_SEED + 8 * step_no,
                                           arena=arena, batch_ids=ids[first:first + sb.shape[0]], seeds_distinct=True)
            return sum(int(h["indices"].numel()) for h in hops), None

    st = Stepper(torch, call, batches, group, device)
    seconds, edges = timed_steps(torch, st, 1, steps, lambda: None, float, min_seconds=0.0, min_repeats=1, max_repeats=1)
    return {"value": edges / seconds[0], "unit": UNIT, "steps": steps, "ms_per_step": seconds[0] / steps * 1e3,
            "edges_per_step": edges / steps, "graph": {"nodes": 100_000, "edges": int(indices.numel())}, "group": group,
            "workload": "GraphSAGE 2-hop uniform sampling, fanouts [10,5], 1,024 seeds/batch, 100,000-node R-MAT graph, "
                        "relabel per hop; seeds from pinned host memory; a step = 1,000 minibatches"}


def secondary_workloads(args, impl, device, indptr, indices):
    """Short legs of the other four configurations, after the headline, on one GPU: each arm runs them with its own
    library (same Python loops).  A leg that fails is reported with its error, never fatal."""
    import torch
    out = {}

    def leg(name, fn):
        t0 = time.time()
        try:
            out[name] = fn()
        except Exception as exc:
            out[name] = {"error": str(exc).splitlines()[0][:200]}
        out[name]["wall_seconds"] = round(time.time() - t0, 1)
        torch.cuda.synchronize()
        torch.cuda.empty_cache()

    leg("small_2hop", lambda: measure_small_sage(torch, impl, device))
    leg("adaptive", lambda: measure_pipeline(torch, "adaptive", impl, device, 40, 5, graph=(indptr, indices)))
    leg("layerwise", lambda: measure_pipeline(torch, "ladies", impl, device, 100, 5))

    def walk():
        m = measure_walk(torch, args, impl, device, steps=3, warmup=1)
        return {"value": m["units"] / m["seconds"], "unit": "walker steps/s", "ms_per_step": m["seconds"] / m["steps"] * 1e3,
                "steps": m["steps"], "graph": m["graph"], "graph_gen_seconds": m["graph_gen_seconds"],
                "walkers": args.walkers, "length": args.walk_length, "checked": m["checked"],
                "checks_pass": m["checks_pass"], "fraction_of_trace_alive": m["fraction_of_trace_alive"],
                "roofline": m["roofline"]}

    leg("random_walk", walk)
    return out


def run_atomics(args):
    """`--workload atomics`: the measurement behind the partitioned unique + relabel — random 64-bit atomicMin on a table
    in a CTA's own shared memory, in the distributed shared memory of clusters of 2 - 16 CTAs, and in L2-resident global
    memory (gsb_selftest_table_atomics).  One JSON line."""
    import ctypes
    import torch
    torch.cuda.set_device(0)
    from graph_sampling_b200 import ops
    ctx = ops.default_context(torch.device("cuda", 0))
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rows = []
    for where, name, clusters in ((0, "own shared memory", (1,)), (1, "distributed shared memory of a cluster", (2, 4, 8, 16)),
                                  (2, "global memory, 32 MB table (L2)", (1,))):
        for c in clusters:
            out = ctypes.c_double(0.0)
            ctx.check(ctx.lib.gsb_selftest_table_atomics(ctx.handle, stream, where, c, 2000, ctypes.byref(out)),
                      "gsb_selftest_table_atomics")
            rows.append({"table": name, "cluster_size": c, "atomics_per_second": out.value})
    print(json.dumps({"metric": "random_64bit_atomic_min_per_second", "unit": "operations/s", "rows": rows,
                      "config": {"workload": "1,024 threads per CTA, one CTA per SM, 200 KB of shared memory per CTA, "
                                             "2,000 rounds of 4 independent atomicMin per thread"}}))


def run_access(args):
    """`--workload access`: what the sampling launches of ONE call of the batched sampler touch, counted exactly from
    the call's own outputs (select_index = the positions it gathered): seed columns and how many are distinct, their
    degrees, the distinct 64-byte lines of `indices` and of `indptr` behind the gathers.  lines x 64 B + the bytes
    written is the least DRAM traffic an order-preserving sampler can cause for these draws (every line fetched once);
    the ratio to the algorithmic bytes is the price of 8-byte gathers in 64-byte DRAM lines, whatever the kernel."""
    import torch
    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    from graph_sampling_b200 import ops
    indptr, indices, batches, batch_ids, info, _ = make_inputs(args, device, 1, 0)
    G = args.group
    ptr = torch.arange(G + 1, dtype=torch.int64, device=device) * BATCH
    hops = ops.sage_sample_batches(indptr, indices, batches[:G].reshape(-1).to(device), ptr, FANOUTS, seed=RUN_SEED,
                                   batch_ids=batch_ids[:G].to(device), seeds_distinct=True)
    deg_all = indptr[1:] - indptr[:-1]
    out = []
    for k, h in zip(FANOUTS, hops):
        seeds, sel = h["seeds"], h["select_index"]
        S, E = int(seeds.numel()), int(sel.numel())
        d = deg_all[seeds]
        lines_idx = int(torch.unique(sel // 8).numel())
        first_line, last_line = (seeds * 8) // 64, (seeds * 8 + 15) // 64        # the indptr pair of a column
        lines_ptr = int(torch.unique(torch.cat([first_line, last_line])).numel())
        visits_ptr = S + int((first_line != last_line).sum())
        alg = 32 * S + 8 + 24 * E
        written = 8 * (S + 1) + 16 * E
        seeds_read = 8 * S
        floor_once = 64 * (lines_idx + lines_ptr) + written + seeds_read          # every line fetched exactly once
        per_visit = 64 * E + 64 * visits_ptr + written + seeds_read                  # every gather its own line
        out.append({"fanout": k, "seed_columns": S, "distinct_seed_columns": int(torch.unique(seeds).numel()),
                    "sampled_edges": E, "mean_degree_of_seed_columns": round(float(d.float().mean()), 1),
                    "share_of_columns_with_degree_le_fanout": round(float((d <= k).float().mean()), 4),
                    "share_of_columns_with_degree_le_64": round(float((d <= 64).float().mean()), 4),
                    "distinct_64B_lines_of_indices": lines_idx, "distinct_64B_lines_of_indptr": lines_ptr,
                    "algorithmic_bytes": alg, "bytes_if_every_distinct_line_is_fetched_once": floor_once,
                    "bytes_if_every_gather_fetches_its_line": per_visit,
                    "floor_over_algorithmic": round(floor_once / alg, 2),
                    "per_gather_over_algorithmic": round(per_visit / alg, 2)})
    print(json.dumps({"metric": "sampler_access_pattern", "graph": info, "minibatches_in_call": G, "batch": BATCH,
                      "hops": out}))


def run_kernels(args):
    """Per-operator throughput on the products-scale graph: every operator of the hot path once, at a size that
    fills the GPU, timed with CUDA events; achieved = algorithmic bytes / time against the measured HBM peak.
    Secondary output (one JSON line with a list)."""
    import torch
    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    from graph_sampling_b200 import ops
    from graph_sampling_b200.synthetic import rmat_csc
    indptr, indices = rmat_csc(args.nodes, args.edges, seed=GRAPH_SEED, symmetric=True, max_degree=MAX_DEGREE,
                               device=device)
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    n = args.nodes
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    peak = float(json.load(open(peaks_path))["hbm_gbs"]) if os.path.exists(peaks_path) else 6650.0
    g = torch.Generator(device=device)
    g.manual_seed(1)
    results = []

    def timed(name, fn, alg_bytes, reps=10, note=""):
        for _ in range(3):
            out = fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            out = fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / reps
        b = alg_bytes(out) if callable(alg_bytes) else alg_bytes
        results.append({"op": name, "ms": round(ms, 4), "algorithmic_MB": round(b / 1e6, 1),
                        "achieved_gbs": round(b / ms / 1e6, 1), "frac": round(b / ms / 1e6 / peak, 4), "note": note})
        return out

    S = 262_144
    seeds = torch.randint(0, n, (S,), generator=g, device=device)
    sl = timed("column slice (count + fill, COO out)", lambda: ops.csc_col_slicing(indptr, indices, seeds, True),
               lambda o: 32 * S + 8 + 32 * o[2].numel(), note="includes one size read-back")
    D = sl[2].numel()
    big = torch.randint(0, n, (2_600_000,), generator=g, device=device)
    timed("fused slice + uniform sample, fanout 10", lambda: ops.fused_csc_col_slicing_sampling(indptr, indices, big, 10, False),
          lambda o: 32 * big.numel() + 8 + 24 * o[1].numel(), note="includes one size read-back")
    sub_indptr, sub_col, sub_row = sl[0], sl[1], sl[2]
    probs = torch.rand(D, generator=g, device=device) + 0.01
    timed("weighted per-column sample, fanout 10", lambda: ops.csc_col_sampling_probs(sub_indptr, sub_row, probs, 10, False, with_coo=False),
          lambda o: 32 * S + 8 + 4 * D + 24 * o[2].numel())
    timed("weighted per-column sample, fanout 64", lambda: ops.csc_col_sampling_probs(sub_indptr, sub_row, probs, 64, False, with_coo=False),
          lambda o: 32 * S + 8 + 4 * D + 24 * o[2].numel(), note="beyond the reference's limit of 32: one CTA per column, radix select")
    items = torch.cat([seeds, sub_row])
    timed("unique + relabel (single table)", lambda: ops.relabel([seeds, sub_row], [sub_row]),
          lambda o: 8 * items.numel() + 8 * o[0].numel() + 8 * D)
    third = sub_row[:1_000_000].contiguous()
    timed("unique + relabel (three arrays: 16-byte slots)", lambda: ops.relabel([seeds, sub_row, third], [sub_row]),
          lambda o: 8 * (items.numel() + third.numel()) + 8 * o[0].numel() + 8 * D,
          note="the general form of gs::Graph::Relabel; two-array calls take the packed-slot kernels above")
    F = 256
    x = torch.randn(n, F, generator=g, device=device)
    xd = x[seeds]
    out = torch.zeros(D, 1, device=device)
    timed("SDDMM dot, F = 256", lambda: ops.sddmm("dot", x, xd, out, 0, 2, sub_row, sub_col), D * (4 * F + 20) + S * 4 * F)
    w = torch.rand(D, generator=g, device=device)
    o1 = torch.zeros(S, device=device)
    timed("segment sum of squares (CSC)", lambda: ops.csc_sum(sub_indptr, None, w, o1, 2), 12 * D + 4 * S)
    o2 = torch.zeros(n, device=device)
    timed("segment sum of squares (COO, atomics)", lambda: ops.coo_sum(sub_row, None, w, o2, 2), 12 * D + 4 * n)
    timed("segment sum of squares (COO, sorted targets)", lambda: ops.coo_sum(sub_col, None, w, o1, 2, targets_in_runs=True), 12 * D + 4 * S,
          note="one atomic per distinct target of a warp")
    o3 = torch.empty(D, device=device)
    timed("segment normalize (CSC)", lambda: ops.csc_normalize(sub_indptr, None, w, o3), 8 * D + 8 * (S + 1))
    rows = torch.randperm(n, generator=g, device=device)[:100_000]
    timed("row slice by membership (CSC)", lambda: ops.csc_row_slicing(sub_indptr, sub_row, rows, True),
          lambda o: 8 * rows.numel() + 8 * D + 24 * o[2].numel())
    timed("CSC -> COO", lambda: ops.csc2coo(sub_indptr, sub_row), 8 * (S + 1) + 8 * D)
    timed("COO -> CSR (stable radix sort)", lambda: ops.coo2csc(sub_col, sub_row, n, False), 32 * D * 3 + 8 * n,
          note="3 radix passes of 32 B per edge")
    lp = torch.rand(1_000_000, generator=g, device=device)
    lp[torch.rand(1_000_000, generator=g, device=device) < 0.5] = 0
    ld = torch.arange(1_000_000, device=device)
    timed("list sampling, 512 of 1 M weighted", lambda: ops.list_sampling(ld, 512, False, probs=lp), 12 * 1_000_000 + 16 * 512,
          note="12 launches; bound by host launch time")
    # ---- feature load, induced subgraph, metapath walk, super-batch operators --------------------------------
    fr = torch.randint(0, n, (1_000_000,), generator=g, device=device)
    timed("feature rows gather, F = 256 (1 M rows)", lambda: ops.gather_rows(x, fr), fr.numel() * (8 + 8 * F))
    timed("edge data gather, F = 1 (13 M of 124 M)", lambda: ops.gather_rows(probs, sub_row % D), D * 16)
    del x, xd
    torch.cuda.empty_cache()
    timed("induced subgraph (262 k columns x 100 k rows)", lambda: ops.csc_col_row_slicing(indptr, indices, seeds, rows),
          lambda o: 32 * S + 8 * rows.numel() + 8 * D + 16 * o[1].numel(), note="two size read-backs")
    wseeds = torch.randint(0, n, (4_000_000,), generator=g, device=device)
    path = [0, 1] * 8
    timed("metapath walk, 4 M walkers x 16 steps, 2 relations", lambda: ops.fused_metapath_random_walk(wseeds, path, [(indptr, indices), (indptr, indices)]),
          wseeds.numel() * (16 + 32 * 16))
    G = 256
    bptr = torch.arange(G + 1, device=device) * (D // G)
    bptr[-1] = D
    sptr = torch.arange(G + 1, device=device) * (S // G)
    timed("BatchUnique, 256 batches", lambda: ops.batch_unique(sub_row, bptr), lambda o: 8 * D + 16 * o[0].numel())
    timed("BatchUnique2 (sorted), 256 batches", lambda: ops.batch_unique(sub_row, bptr, sort=True),
          lambda o: 8 * D + 16 * o[0].numel() + 5 * 24 * D, note="5 keys-only radix passes of 24 B per item")
    bcol = seeds[sub_col]
    timed("BatchCOORelabel, 256 batches", lambda: ops.batch_coo_relabel(seeds, sptr, bcol, sub_row, bptr),
          lambda o: 8 * (S + D) + 8 * o[0].numel() + 8 * D + 16 * D)
    timed("BatchCSRRelabel, 256 batches", lambda: ops.batch_csr_relabel(seeds, sptr, sub_row, bptr),
          lambda o: 8 * (S + D) + 8 * o[0].numel() + 8 * D,
          note="the generic entry of the batched unique + relabel: counting pass + partitioned form")
    rptr = torch.arange(G + 1, device=device) * (rows.numel() // G)
    rows_m = rows[:int(rows.numel() // G) * G].contiguous()   # the offsets must cover the whole member array
    timed("BatchCOOSlicing by membership, 256 batches", lambda: ops.batch_coo_slicing(1, sub_row, sub_col, bptr, rows_m, rptr),
          lambda o: 8 * rows_m.numel() + 16 * D + 16 * o[0].numel())
    enc = timed("BatchEncode", lambda: ops.batch_encode(sub_row, bptr, n), 16 * D)
    timed("GetBatchOffsets + decode", lambda: ops.get_batch_offsets(enc, G, n), 16 * D)
    timed("BatchConcat of 2 arrays", lambda: ops.batch_concat([seeds, sub_row], [sptr, bptr]), 24 * (S + D))
    timed("segmented list sampling, 256 x 4000 of 13 M", lambda: ops.batch_list_sampling_probs(probs, 4000, False, bptr),
          12 * D + 8 * 4000 * G, note="two histogram passes, then only the candidates are sorted")
    print(json.dumps({"metric": "per_operator_roofline", "unit": "GB/s", "peak": peak, "graph": {"nodes": n, "edges": int(indices.numel())},
                      "operators": results}))


def run_kernels_reference(args):
    """The reference's own CUDA operators (unmodified sources compiled for sm_100) on the inputs of run_kernels,
    timed the same way: the per-operator counterpart of `--impl reference`.  Secondary output."""
    import torch
    lib = os.path.join(ROOT, "oracle", "_ref", "libgs_ref.so")
    if not os.path.exists(lib):
        print(json.dumps({"metric": "per_operator_time", "impl": "reference",
                          "unavailable": "oracle/_ref/libgs_ref.so is not built (oracle/build_ref.sh)"}))
        return
    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    from graph_sampling_b200.synthetic import rmat_csc
    torch.classes.load_library(lib)
    Graph, ops = torch.classes.gs_classes.Graph, torch.ops.gs_ops
    indptr, indices = rmat_csc(args.nodes, args.edges, seed=GRAPH_SEED, symmetric=True, max_degree=MAX_DEGREE,
                               device=device)
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    n = args.nodes
    _COO, _CSC, _CSR = 1, 2, 4
    g = torch.Generator(device=device)
    g.manual_seed(1)
    results = []

    def timed(name, fn, reps=10):
        try:
            for _ in range(3):
                out = fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                out = fn()
            e1.record()
            torch.cuda.synchronize()
            results.append({"op": name, "ms": round(e0.elapsed_time(e1) / reps, 4)})
            return out
        except Exception as exc:  # an operator the reference cannot run at this size is reported, not fatal
            results.append({"op": name, "ms": None, "error": str(exc).splitlines()[0][:120]})
            return None

    A = Graph(False)
    A._CAPI_LoadCSC(indptr, indices)
    S = 262_144
    seeds = torch.randint(0, n, (S,), generator=g, device=device)
    sub = timed("column slice (count + fill, COO out)", lambda: A._CAPI_Slicing(seeds, 0, _CSC, _CSC + _COO, False))
    big = torch.randint(0, n, (2_600_000,), generator=g, device=device)
    timed("fused slice + uniform sample, fanout 10", lambda: A._CAPI_FusedColumnwiseSlicingSampling(big, 10, False))
    sub_indptr, sub_row, _ = sub._CAPI_GetCSC()
    sub_col = sub._CAPI_GetCOO()[1]
    D = sub_row.numel()
    probs = torch.rand(D, generator=g, device=device) + 0.01
    timed("weighted per-column sample, fanout 10", lambda: sub._CAPI_SamplingWithProbs(0, probs, 10, False, _CSC, _CSC))
    timed("unique + relabel (single table)", lambda: sub._CAPI_Relabel())
    F = 256
    x = torch.randn(n, F, generator=g, device=device)
    xd = x[seeds]
    out = torch.zeros(D, 1, device=device)
    timed("SDDMM dot, F = 256", lambda: sub._CAPI_SDDMM("dot", x, xd, out, 0, 2, _COO))
    w = torch.rand(D, generator=g, device=device)
    sub._CAPI_SetData(w)
    timed("segment sum of squares (CSC)", lambda: sub._CAPI_Sum(0, 2, _CSC))
    timed("segment sum of squares (COO, atomics)", lambda: sub._CAPI_Sum(1, 2, _COO))
    timed("segment sum of squares (COO, sorted targets)", lambda: sub._CAPI_Sum(0, 2, _COO))
    timed("segment normalize (CSC)", lambda: sub._CAPI_Normalize(0, _CSC))
    rows = torch.randperm(n, generator=g, device=device)[:100_000]
    timed("row slice by membership (CSC)", lambda: sub._CAPI_Slicing(rows, 1, _CSC, _CSC + _COO, False))
    lp = torch.rand(1_000_000, generator=g, device=device)
    lp[torch.rand(1_000_000, generator=g, device=device) < 0.5] = 0
    ld = torch.arange(1_000_000, device=device)
    timed("list sampling, 512 of 1 M weighted", lambda: ops._CAPI_ListSamplingWithProbs(ld, lp, 512, False))
    fr = torch.randint(0, n, (1_000_000,), generator=g, device=device)
    timed("feature rows gather, F = 256 (1 M rows)", lambda: x[fr])    # the reference indexes with torch here
    del x, xd
    torch.cuda.empty_cache()
    timed("induced subgraph (262 k columns x 100 k rows)", lambda: A._CAPI_FusionSlicing(seeds, rows))
    G = 256
    bptr = torch.arange(G + 1, device=device) * (D // G)
    bptr[-1] = D
    sptr = torch.arange(G + 1, device=device) * (S // G)
    timed("BatchUnique, 256 batches", lambda: ops._CAPI_BatchUnique(sub_row, bptr))
    timed("BatchUnique2 (sorted), 256 batches", lambda: ops._CAPI_BatchUnique2(sub_row, bptr))
    bcol = seeds[sub_col]
    timed("BatchCOORelabel, 256 batches", lambda: ops._CAPI_BatchCOORelabel(seeds, sptr, bcol, sub_row, bptr))
    timed("BatchCSRRelabel, 256 batches", lambda: ops._CAPI_BatchCSRRelabel(seeds, sptr, sub_row, bptr))
    rptr = torch.arange(G + 1, device=device) * (rows.numel() // G)
    rows_m = rows[:int(rows.numel() // G) * G].contiguous()   # the offsets must cover the whole member array
    timed("BatchCOOSlicing by membership, 256 batches", lambda: ops._CAPI_BatchCOOSlicing(1, sub_row, sub_col, bptr, rows_m, rptr))
    enc = timed("BatchEncode", lambda: ops._CAPI_BatchEncode(sub_row, bptr, n))
    if enc is not None:
        timed("GetBatchOffsets + decode", lambda: ops._CAPI_GetBatchOffsets(enc, G, n))
    timed("BatchConcat of 2 arrays", lambda: ops._CAPI_BatchConcat([seeds, sub_row], [sptr, bptr]))
    timed("segmented list sampling, 256 x 4000 of 13 M", lambda: ops._CAPI_BatchListSamplingWithProbs(probs, 4000, False, bptr))
    print(json.dumps({"metric": "per_operator_time", "unit": "ms", "impl": "reference",
                      "graph": {"nodes": n, "edges": int(indices.numel())}, "operators": results}))


if __name__ == "__main__":
    a = parse()
    if a.workload == "kernels":
        run_kernels_reference(a) if a.impl == "reference" else run_kernels(a)
    elif a.workload == "walk":
        run_walk(a)
    elif a.workload == "access":
        run_access(a)
    elif a.workload == "atomics":
        run_atomics(a)
    elif a.workload in ("ladies", "adaptive"):
        run_pipeline(a)
    elif a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)
