#!/usr/bin/env python
"""Benchmark of the attention hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one decode step of the Llama-2-7B-shaped paged workload (batch 64, 32 MHA heads,
head size 128, block size 16, contexts uniform in [512, 4096], 16384-block pool): the cache
write of the 64 new tokens (reshape_and_cache) followed by decode attention over the paged
cache (paged_attention_v1).  With N > 1 the KV heads are split over the ranks (tensor-parallel
layout) and the head outputs are gathered inside the step (stored into every rank's buffer by the
attention call itself, or all-gathered over NCCL with --gather nccl), so the total work is fixed
("strong" scaling).  The metric is the achieved HBM traffic rate in TB/s computed from
the ALGORITHMIC bytes of the step (K and V once per (sequence, kv head), q, out, block tables,
context lengths, and the cache write), aggregated over all ranks.  The timed steps are submitted
as CUDA-graph replays, four steps to a graph (--steps-per-graph), each step one library call.

The line also carries the long-context causal prefill throughput (2 x 32768 tokens, 64 q / 8 kv
heads) in TFLOP/s under "prefill", the roofline of the dominant decode kernel, an end-to-end
figure through the public API with host buffers, device time and roofline fraction of the other
configurations (GQA decode, the mixed step's decode, prefill chunks, cache write and fork copy)
under "configs", the parity of every timed output against the CPU oracle on sampled rows (and, on
more than one GPU, bit equality of the fused gather with an NCCL gather) under "parity" -- the run
exits non-zero when a bound is exceeded -- and the CPU baseline: the PyTorch-CPU port of rLLM's own
CPU kernels timed on the same workload.

--impl reference times that CPU port (the reference's CPU path for this operation; its Rust
original cannot be built in this image) with all host threads, on rank 0 only.
"""
import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

METRIC = "paged-decode attn HBM TB/s (prefill attn TFLOPS under 'prefill')"
UNIT = "TB/s"
WORKLOAD = "decode_llama2_7b_b64_mha32_d128_bs16_ctx512-4096_pool16384+reshape_and_cache_64"
MAX_ABS, MEAN_ABS = 2e-2, 2e-3  # bf16 attention outputs against the fp32-softmax oracle
L2_BYTES = 126 << 20
# Bytes a GPU should stream before it meets the same cache line again, so that HBM and not L2 is
# measured: when one step reads less than this per GPU (kv-head shards of 4 and 8 GPUs), the bench
# keeps several copies of the KV pool and the steps walk through them in turn.
MIN_STREAM_BYTES = 1 << 30
# DRAM bytes (read + write) of paged_decode_kernel per algorithmic byte, from ncu captures of one
# launch of rank 0's shard at each world size (`--profile decode --profile-world N`; world size 1:
# the 16-sequence case of `--profile decode`; traffic grows in proportion to the tokens read).  The
# summaries are under profiles/.  A world size without a capture reports no traffic figure.
DECODE_TRAFFIC_RATIO = {1: 1.012, 2: 1.007, 4: 1.010, 8: 1.015}
# DRAM bytes (read + write) of one full-size varlen_prefill_kernel launch (2 x 32768, 64/8 heads) on
# one GPU: a one-pass ncu capture of `--profile prefill_full` (15.93 GB read, 1.18 GB written, for
# 2.42 GB of q, k, v and output: the two sequences' K/V, 268 MB, do not fit the L2 and are fetched
# again by later row tiles; 0.58 TB/s, 9 % of the HBM rate).  Shards of 2, 4, 8 GPUs were not captured.
PREFILL_TRAFFIC_BYTES = {1: 17.11e9}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def shared_config(n_gpus, step_bytes):
    """The part of the JSON line that names the workload: the same in both arms."""
    return {"workload": WORKLOAD, "sharding": "kv-heads/%d" % n_gpus,
            "algorithmic_bytes_per_step": int(step_bytes),
            "l2": "inputs larger than L2: every step streams the K/V of all 64 sequences (2.4 GB over all "
                  "GPUs); where a GPU's share is below 1 GB, consecutive steps read different copies of the pool"}


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML (read-only) while a timed region runs:
    `region(name)` opens a region, `region(None)` closes it; samples outside a region are dropped."""

    def __init__(self, index, period=0.005):
        super().__init__(daemon=True)
        self.index, self.period = index, period
        self.data, self.current, self.max_mhz = {}, None, None
        self._stop_evt = threading.Event()
        self.ok = False
        try:
            import pynvml
            self.nv = pynvml
            pynvml.nvmlInit()
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
            self.ok = True
        except Exception:
            self.ok = False

    def region(self, name):
        self.current = name

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
            cur = self.current
            if cur is not None:
                try:
                    mhz = int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                    r = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
                    samples, reasons = self.data.setdefault(cur, ([], set()))
                    samples.append(mhz)
                    for bit, name in names.items():
                        if r & bit:
                            reasons.add(name)
                except Exception:
                    pass
            time.sleep(self.period)

    def stop(self):
        self._stop_evt.set()
        if self.is_alive():
            self.join(timeout=2)

    def summary(self, name):
        samples, reasons = self.data.get(name, ([], set()))
        if not samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(reasons), "samples": 0}
        return {"sm_mhz": int(statistics.median(samples)), "sm_min_mhz": min(samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(reasons), "samples": len(samples)}


def physical_gpu_index(local_rank):
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except Exception:
            return local_rank
    return local_rank


# ---------------------------------------------------------------------------------------------
# CPU arm: the PyTorch-CPU port of rLLM's CPU kernels on the same workload
# ---------------------------------------------------------------------------------------------
def cpu_inputs(n_seqs=64):
    """The decode workload's first n_seqs sequences (all 64 by default) with their blocks compacted
    into an fp32 pool (the CPU build of rLLM runs fp32).  Contexts and tables are the benchmark's own;
    the pool holds the blocks in use (the GPU arm's 16384-block pool is mostly free blocks)."""
    import workloads
    ctx = workloads.draw_context_lens("uniform", 64, 512, 4096, 2001)[:n_seqs]
    hkv = hq = 32
    nblk = sum((c + 15) // 16 for c in ctx)
    g = torch.Generator().manual_seed(2003)
    kc = torch.randn(nblk, hkv, 16, 16, 8, generator=g)
    vc = torch.randn(nblk, hkv, 128, 16, generator=g)
    q = torch.randn(n_seqs, hq, 128, generator=g)
    table, _ = workloads.build_block_tables(ctx, nblk, 2002)
    nk = torch.randn(n_seqs, hkv, 128, generator=g)
    nv = torch.randn(n_seqs, hkv, 128, generator=g)
    slots = torch.tensor([int(table[i, (c - 1) // 16]) * 16 + (c - 1) % 16 for i, c in enumerate(ctx)],
                         dtype=torch.int32)
    kv = sum(ctx) * 2 * hkv * 128 * 2
    qo = n_seqs * hq * 128 * 2 * 2
    bt = sum((c + 15) // 16 for c in ctx) * 4 + 4 * n_seqs
    cw = n_seqs * hkv * 128 * 2 * 2 * 2
    return dict(q=q, kc=kc, vc=vc, table=table, ctx=torch.tensor(ctx, dtype=torch.int32), nk=nk, nv=nv,
                slots=slots, hkv=hkv, bytes=kv + qo + bt + cw, n_seqs=n_seqs)


def cpu_step(c):
    from oracle import refkernels_cpu as R
    R.reshape_and_cache(c["nk"], c["nv"], c["kc"], c["vc"], c["slots"])
    return R.decode_step_cpu(c["q"], c["kc"], c["vc"], c["hkv"], 1.0 / 128 ** 0.5, c["table"], c["ctx"], 16)


def time_cpu(steps, warmup, n_seqs=64, budget_s=240.0):
    """Times the CPU port on the whole workload.  The first warm-up step is also a probe: if
    steps + warmup such steps would take more than budget_s, the sample shrinks to the first
    sequences that fit (and the JSON line says so), so that any --steps/--warmup ends in minutes."""
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    c = cpu_inputs(n_seqs)
    t0 = time.perf_counter()
    cpu_step(c)
    probe = time.perf_counter() - t0
    if probe * (steps + warmup) > budget_s and n_seqs > 8:
        n_seqs = max(8, int(n_seqs * budget_s / (probe * (steps + warmup))))
        c = cpu_inputs(n_seqs)
        cpu_step(c)
    for _ in range(max(0, warmup - 1)):
        cpu_step(c)
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_step(c)
    dt = (time.perf_counter() - t0) / max(steps, 1)
    what = "all 64 sequences" if n_seqs == 64 else "first %d of the 64 sequences" % n_seqs
    return {"value": c["bytes"] / dt / 1e12, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": "%s of the workload (%.1f MB algorithmic per step), %d timed steps, fp32, "
                      "gather_cached_kv + repeat_kv + per-sequence scaled_dot_product_attention as in "
                      "refkernels.rs, %.3f s per step" % (what, c["bytes"] / 1e6, steps, dt)}, dt, c["bytes"]


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps, warm = max(1, args.steps), max(1, args.warmup)
    cb, dt, step_bytes = time_cpu(steps, warm)
    line = {
        "impl": "reference", "metric": METRIC, "value": cb["value"], "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": warm, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": shared_config(args.gpus, step_bytes),
        "note": "CPU path of the reference (refkernels.rs port; the Rust original cannot be built in this "
                "image), whole workload per step, all host threads, rank 0 only",
        "cpu_baseline": cb,
        "e2e": {"value": cb["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------------
# Parity checks (after the timed regions, never inside them): the CPU oracle as the checker
# ---------------------------------------------------------------------------------------------
def decode_parity(full, gathered, n_pick=8):
    """Gathered decode output [S, Hq, 128] against the fp32-softmax oracle on the n_pick shortest and
    n_pick longest sequences, all heads.  `full` is the UNSHARDED workload (same seed) on the GPU,
    with the step's new tokens not yet written; their blocks are compacted onto the CPU, the new
    tokens are written there by the oracle's reshape_and_cache, then the oracle attends."""
    from oracle import cpu_oracle as O
    ctx = full.context_list
    order = sorted(range(len(ctx)), key=lambda i: ctx[i])
    pick = order[:n_pick] + order[-n_pick:] if len(ctx) > 2 * n_pick else list(range(len(ctx)))
    tables = full.block_tables.cpu()
    rows = [tables[i, :(ctx[i] + 15) // 16].tolist() for i in pick]
    flat = torch.tensor([b for r in rows for b in r], dtype=torch.int64, device=full.key_cache.device)
    kc = full.key_cache[flat].cpu()
    vc = full.value_cache[flat].cpu()
    width = max(len(r) for r in rows)
    bt = torch.zeros(len(pick), width, dtype=torch.int32)
    pos, slots = 0, []
    for j, r in enumerate(rows):
        bt[j, :len(r)] = torch.arange(pos, pos + len(r), dtype=torch.int32)
        c = ctx[pick[j]]
        slots.append((pos + (c - 1) // 16) * 16 + (c - 1) % 16)
        pos += len(r)
    sel = torch.tensor(pick, dtype=torch.int64)
    O.reshape_and_cache(full.new_key.cpu()[sel].contiguous(), full.new_value.cpu()[sel].contiguous(), kc, vc,
                        torch.tensor(slots, dtype=torch.int32))
    cl = torch.tensor([ctx[i] for i in pick], dtype=torch.int32)
    want = O.paged_attention_v1(full.query.cpu()[sel].contiguous(), kc, vc, full.num_kv_heads, full.scale, bt, cl)
    mx, mean = O.error_stats(gathered.cpu()[sel], want)
    return [mx, mean], len(pick)


def prefill_parity(full, gathered, n_rows=512, seed=77):
    """Gathered prefill output [total_q, Hq, 128] against the oracle on n_rows random
    (sequence, row, head) triples plus the first and last row of every sequence."""
    from oracle import cpu_oracle as O
    g = torch.Generator().manual_seed(seed)
    hq = full.q.shape[1]
    cu = full.cu_seqlens_q.cpu().tolist()
    trip = []
    for b in range(len(cu) - 1):
        for t in (cu[b], cu[b + 1] - 1):
            trip.append((b, t, int(torch.randint(0, hq, (1,), generator=g))))
    while len(trip) < n_rows:
        b = int(torch.randint(0, len(cu) - 1, (1,), generator=g))
        t = int(torch.randint(cu[b], cu[b + 1], (1,), generator=g))
        trip.append((b, t, int(torch.randint(0, hq, (1,), generator=g))))
    rows = torch.tensor(trip, dtype=torch.int32)
    want = O.flash_attn_varlen_rows(full.q.cpu(), full.k.cpu(), full.v.cpu(), full.cu_seqlens_q.cpu(),
                                    full.cu_seqlens_k.cpu(), rows, full.scale, True)
    idx_t = rows[:, 1].to(torch.int64).to(gathered.device)
    idx_h = rows[:, 2].to(torch.int64).to(gathered.device)
    got = gathered[idx_t, idx_h].cpu()
    mx, mean = O.error_stats(got, want)
    return [mx, mean], len(trip)


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------
class Runner:
    """Process-wide pieces of one bench run: device, ranks, peaks, timing helpers."""

    def __init__(self, args):
        import torch.distributed as dist
        self.dist = dist
        self.args = args
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        if self.world != args.gpus and self.world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node %d" % args.gpus)
        self.dev = torch.device("cuda", self.local_rank)
        torch.cuda.set_device(self.dev)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.dev)
        self.peaks = load_peaks()
        import workloads
        self.shard = workloads.Shard(rank=self.rank, world=self.world)
        self.flush_buf = None

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(self, x):
        if self.world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=self.dev)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def all_true(self, ok):
        if self.world == 1:
            return bool(ok)
        t = torch.tensor([1 if ok else 0], dtype=torch.int32, device=self.dev)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MIN)
        return bool(int(t.item()))

    def flush(self):
        """Writes a buffer of four times the L2 size."""
        if self.flush_buf is None:
            self.flush_buf = torch.empty(4 * L2_BYTES, dtype=torch.uint8, device=self.dev)
        self.flush_buf.zero_()

    def capture(self, fn):
        """fn's launches as a CUDA graph (one eager run first, on the capture stream, so that lazily
        sized scratch exists before the capture)."""
        side = torch.cuda.Stream(self.dev)
        side.wait_stream(torch.cuda.current_stream(self.dev))
        with torch.cuda.stream(side):
            fn()
        torch.cuda.current_stream(self.dev).wait_stream(side)
        self.barrier()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            fn()
        return g

    def time_rotating(self, fns, reps, warm=2):
        """Device time (ms) of ONE launch: the calls in `fns` -- the same operation on distinct
        buffer sets whose sizes add up to several times the L2, so that every launch finds its
        data in HBM -- are captured back to back into one CUDA graph, the graph is replayed `reps`
        times between two events, and the elapsed time is divided by the number of launches.  Max
        over ranks.  Timing a run of launches instead of one keeps the cost of recording an event
        and starting a graph (several microseconds) out of kernels that take ten."""
        def all_once():
            for f in fns:
                f()
        g = self.capture(all_once)
        for _ in range(warm):
            g.replay()
        self.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            g.replay()
        b.record()
        self.barrier()
        return self.max_over_ranks(a.elapsed_time(b)) / (reps * len(fns))


def copies_to_stream(nbytes, at_least=MIN_STREAM_BYTES, cap=32):
    """How many distinct buffer sets of nbytes a run of launches needs to stream at_least bytes."""
    n = 1
    while n * nbytes < at_least and n < cap:
        n += 1
    return n


def roof(kind, work_local, ms, peaks, extra=None):
    if kind == "hbm":
        ach, peak, unit = work_local / (ms * 1e-3) / 1e9, peaks["hbm_gbs"], "GB/s"
    else:
        ach, peak, unit = work_local / (ms * 1e-3) / 1e12, peaks["bf16_tflops_sustained"], "TFLOP/s"
    row = {"ms": ms, "bound": "hbm" if kind == "hbm" else "tensor", "achieved": ach, "unit": unit,
           "peak": peak, "frac": ach / peak, "work_per_gpu": work_local}
    if kind != "hbm":
        row["frac_of_burst_peak"] = ach / peaks["bf16_tflops"]
    if extra:
        row.update(extra)
    return row


def run_ours(args):
    from aici_b200 import tch_cuda, _lib, sharding
    import workloads
    R = Runner(args)
    dist, dev, world, rank, peaks, shard = R.dist, R.dev, R.world, R.rank, R.peaks, R.shard

    # ---- decode workload ------------------------------------------------------------------
    w = workloads.decode_llama2_7b(dev, shard=shard)
    S, hq_local = w.query.shape[0], w.query.shape[1]
    hq_total = hq_local * world
    out = torch.empty_like(w.query)
    gathered = torch.empty(world, S, hq_local, 128, dtype=torch.bfloat16, device=dev) if world > 1 else None
    step_bytes_local = w.algorithmic_bytes() + w.cache_write_bytes()
    decode_bytes_local = w.algorithmic_bytes()
    # pools: copies of this rank's KV pool that consecutive steps read in turn (see MIN_STREAM_BYTES)
    n_pools = 1
    while n_pools * decode_bytes_local < MIN_STREAM_BYTES and n_pools < 8:
        n_pools *= 2
    pools = [(w.key_cache, w.value_cache)] + [(w.key_cache.clone(), w.value_cache.clone())
                                              for _ in range(n_pools - 1)]
    fused = world > 1 and args.gather == "fused"
    pg, fused_fallback, peer_kind = None, None, 0
    if fused:
        # peer-mapped output buffers through the library's own calls (CUDA IPC); if any rank cannot
        # set them up, every rank falls back to the NCCL gather (and the JSON line says so)
        try:
            pg = sharding.PeerGather(S, hq_total, 128, dev, buffers=2)
            pg.barrier()
            peer_kind = pg.mem.kind
        except Exception as e:  # noqa: BLE001
            fused_fallback = "%s: %s" % (type(e).__name__, str(e)[:160])
            fused, pg = False, None

    def attention(q, bt, cl, pool, buf):
        """decode attention + head gather: fused epilogue (peer stores, barrier folded into the last
        kernel) into output buffer `buf`, or an NCCL all-gather"""
        kc, vc = pools[pool]
        if fused:
            tch_cuda.paged_attention_v1_peers(pg._ptrs[buf], hq_total, pg.head0, q, kc, vc, w.num_kv_heads,
                                              w.scale, bt, cl, 16, w.max_context_len,
                                              barrier_flags=pg.flag_ptrs, rank=pg.rank)
            return pg.tensors[buf]
        tch_cuda.paged_attention_v1(out, q, kc, vc, w.num_kv_heads, w.scale, bt, cl, 16, w.max_context_len, None)
        if world > 1:
            dist.all_gather_into_tensor(gathered.view(-1, hq_local, 128), out)
            return gathered
        return out

    def full_step(nk, nv, slots, q, bt, cl, pool, buf):
        """One decode step: cache write of the new tokens + decode attention + head gather.  By default
        one library call (aici_decode_step: same two kernels, the decode grid streams everything but the
        sequences' last tiles while the cache write runs); --separate-calls makes the two crate calls."""
        kc, vc = pools[pool]
        if args.separate_calls:
            tch_cuda.reshape_and_cache(nk, nv, kc, vc, slots)
            return attention(q, bt, cl, pool, buf)
        if fused:
            tch_cuda.decode_step(None, nk, nv, slots, q, kc, vc, w.num_kv_heads, w.scale, bt, cl, 16,
                                 w.max_context_len, peer_ptrs=pg._ptrs[buf], barrier_flags=pg.flag_ptrs,
                                 rank=pg.rank, total_heads=hq_total, head0=pg.head0)
            return pg.tensors[buf]
        tch_cuda.decode_step(out, nk, nv, slots, q, kc, vc, w.num_kv_heads, w.scale, bt, cl, 16, w.max_context_len)
        if world > 1:
            dist.all_gather_into_tensor(gathered.view(-1, hq_local, 128), out)
            return gathered
        return out

    def step(i=0):
        return full_step(w.new_key, w.new_value, w.slot_mapping, w.query, w.block_tables, w.context_lens,
                         i % n_pools, i % 2)

    # a graph per (pool, output buffer) combination; step i replays graph i mod n_graphs
    n_graphs = max(n_pools, 2 if fused else 1)
    use_graph = (world == 1 or fused) and not args.no_graph
    sampler = ClockSampler(physical_gpu_index(R.local_rank))
    sampler.start()
    for i in range(args.warmup):
        step(i)
    R.barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    prof = torch.cuda.cudart() if args.profile_step is not None else None

    def timed_steps(runs, steps, profile=False, group=None):
        """`steps` back-to-back steps between two events -> (device ms, host wall ms).  With
        `profile`, one step is bracketed by the profiler API (cudaProfilerStart/Stop, as rLLM's
        --profile-step does around one forward pass, so that a capture can be limited to it).
        `group` = (replay, n): one graph that holds n consecutive steps, used for as many whole
        groups as fit; the remaining steps go one by one."""
        R.barrier()
        t0 = time.perf_counter()
        ev0.record()
        i = 0
        while i < steps:
            if group is not None and i + group[1] <= steps:
                group[0]()
                i += group[1]
                continue
            mark = profile and prof is not None and i == args.profile_step
            if mark:
                prof.cudaProfilerStart()
            runs[i % len(runs)]()
            if mark:
                prof.cudaProfilerStop()
            i += 1
        ev1.record()
        ev1.synchronize()
        wall = (time.perf_counter() - t0) * 1e3
        R.barrier()
        return ev0.elapsed_time(ev1), wall

    if use_graph:
        graphs = [R.capture(lambda i=i: step(i)) for i in range(n_graphs)]
        runs = [g.replay for g in graphs]
    else:
        runs = [(lambda i=i: step(i)) for i in range(n_graphs)]
    # The forward pass of a model issues one such step per layer inside one graph; the timed steps
    # are submitted the same way, several to a graph (a whole number of turns through the pools and
    # output buffers), unless one step is to be bracketed for a profiler.
    spg = args.steps_per_graph if args.steps_per_graph > 0 else max(n_graphs, 4)
    if spg > 1:
        spg = (spg + n_graphs - 1) // n_graphs * n_graphs
    group = None
    if use_graph and spg > 1 and args.profile_step is None:
        group = (R.capture(lambda: [step(i) for i in range(spg)]).replay, spg)
    else:
        spg = 1
    for i in range(3 * n_graphs):
        runs[i % n_graphs]()
    if group is not None:
        for _ in range(2):
            group[0]()
    sampler.region("decode")
    ms_total = R.max_over_ranks(timed_steps(runs, args.steps, profile=True, group=group)[0])
    ms_step = ms_total / args.steps

    # The decode call alone (decode + merge launches; with the fused gather their stores to the
    # peers and the barrier in the merge kernel's tail), for the roofline: back-to-back replays of
    # graphs holding just that call, so the figure is device time.
    def attention_only(i=0):
        return attention(w.query, w.block_tables, w.context_lens, i % n_pools, i % 2)

    if use_graph:
        a_runs = [R.capture(lambda i=i: attention_only(i)).replay for i in range(n_graphs)]
    else:
        a_runs = [(lambda i=i: attention_only(i)) for i in range(n_graphs)]
    a_group = None
    if group is not None:
        a_group = (R.capture(lambda: [attention_only(i) for i in range(spg)]).replay, spg)
        a_group[0]()
    for i in range(3 * n_graphs):
        a_runs[i % n_graphs]()
    att_ms = R.max_over_ranks(timed_steps(a_runs, args.steps, group=a_group)[0]) / args.steps
    sampler.region(None)
    status = _lib.last_status()
    if status != 0:
        raise SystemExit("device status word is %d after the timed region" % status)
    value = step_bytes_local * world / (ms_step * 1e-3) / 1e12
    achieved_gbs = decode_bytes_local / (att_ms * 1e-3) / 1e9

    # ---- end to end through the public API with host buffers -------------------------------
    # The step's inputs (q, new k/v, slot map, block tables, context lens) sit in ONE page-locked
    # staging buffer at 256-byte aligned offsets and reach the device with ONE copy per step into a
    # buffer of the same layout; the kernels read views of it; the gathered output is read back.
    parts = {"q": w.query, "nk": w.new_key, "nv": w.new_value, "slots": w.slot_mapping,
             "bt": w.block_tables, "cl": w.context_lens}
    offs, cur = {}, 0
    for k, t in parts.items():
        offs[k] = cur
        cur = (cur + t.numel() * t.element_size() + 255) // 256 * 256
    staging = torch.empty(cur, dtype=torch.uint8).pin_memory()
    dev_in = torch.empty(cur, dtype=torch.uint8, device=dev)

    def section(buf, k):
        t = parts[k]
        n = t.numel() * t.element_size()
        return buf[offs[k]:offs[k] + n].view(t.dtype).view(t.shape)
    for k, t in parts.items():
        section(staging, k).copy_(t.cpu())
    d = {k: section(dev_in, k) for k in parts}
    host_out = torch.empty((S, hq_total, 128) if world > 1 else out.shape, dtype=out.dtype).pin_memory()
    h2d = sum(t.numel() * t.element_size() for t in parts.values())
    d2h = host_out.numel() * host_out.element_size()

    def e2e_step(i=0):
        dev_in.copy_(staging, non_blocking=True)
        o = full_step(d["nk"], d["nv"], d["slots"], d["q"], d["bt"], d["cl"], i % n_pools, i % 2)
        if world > 1 and not fused:
            o = o.permute(1, 0, 2, 3).reshape(S, hq_total, 128)
        host_out.copy_(o, non_blocking=True)

    for i in range(max(3, args.warmup // 2)):
        e2e_step(i)
    R.barrier()
    if use_graph:
        e_runs = [R.capture(lambda i=i: e2e_step(i)).replay for i in range(n_graphs)]
    else:
        e_runs = [(lambda i=i: e2e_step(i)) for i in range(n_graphs)]
    e_group = None
    if group is not None:
        e_group = (R.capture(lambda: [e2e_step(i) for i in range(spg)]).replay, spg)
        e_group[0]()
    for i in range(3 * n_graphs):
        e_runs[i % n_graphs]()
    e2e_dev_ms, e2e_wall = timed_steps(e_runs, args.steps, group=e_group)
    e2e_ms = R.max_over_ranks(max(e2e_dev_ms, e2e_wall)) / args.steps  # the slower of device and host clocks
    e2e_wall_ms = R.max_over_ranks(e2e_wall) / args.steps
    e2e_value = step_bytes_local * world / (e2e_ms * 1e-3) / 1e12

    # ---- parity of the timed decode step (outside the timed regions) --------------------------
    parity = {}
    last = step(0)
    torch.cuda.synchronize()
    dec_gathered = last if (world == 1 or fused) else last.permute(1, 0, 2, 3).reshape(S, hq_total, 128)
    if world > 1:
        # the fused gather against one NCCL gather of the same step, bit for bit, on every rank
        tch_cuda.paged_attention_v1(out, w.query, w.key_cache, w.value_cache, w.num_kv_heads, w.scale,
                                    w.block_tables, w.context_lens, 16, w.max_context_len, None)
        via_nccl = sharding.gather_heads(out).contiguous()
        same = torch.equal(dec_gathered.contiguous().view(torch.int16), via_nccl.view(torch.int16))
        parity["fused_equals_nccl"] = R.all_true(same) if fused else None
    dec_gathered = dec_gathered.clone()
    del pools
    w.key_cache = w.value_cache = None
    torch.cuda.empty_cache()
    if rank == 0:
        full = workloads.decode_llama2_7b(dev)
        parity["decode"], parity["decode_sequences_checked"] = decode_parity(full, dec_gathered)
        del full
    torch.cuda.empty_cache()

    # ---- the other configurations: device time per launch over rotating buffer sets ------------
    configs = {}
    reps = max(5, min(args.steps, 20))
    if not args.headline_only:
        for key, make in (("cfg3", workloads.decode_llama3_8b), ("cfg5_decode", workloads.decode_mixed_step)):
            cw = make(dev, shard=shard)
            tch_cuda.reshape_and_cache(cw.new_key, cw.new_value, cw.key_cache, cw.value_cache, cw.slot_mapping)
            n_sets = copies_to_stream(cw.algorithmic_bytes())
            cpools = [(cw.key_cache, cw.value_cache)] + [(cw.key_cache.clone(), cw.value_cache.clone())
                                                         for _ in range(n_sets - 1)]
            o_loc = torch.empty_like(cw.query)
            cpg = None
            if fused:
                cpg = sharding.PeerGather(cw.query.shape[0], cw.num_heads * world, 128, dev, buffers=2)
                cpg.barrier()

            def dec(i, cw=cw, o_loc=o_loc, cpg=cpg, cpools=cpools):
                kc_, vc_ = cpools[i % len(cpools)]
                if cpg is not None:
                    tch_cuda.paged_attention_v1_peers(cpg._ptrs[i % 2], cw.num_heads * world, cpg.head0, cw.query,
                                                      kc_, vc_, cw.num_kv_heads, cw.scale, cw.block_tables,
                                                      cw.context_lens, 16, cw.max_context_len,
                                                      barrier_flags=cpg.flag_ptrs, rank=cpg.rank)
                else:
                    tch_cuda.paged_attention_v1(o_loc, cw.query, kc_, vc_, cw.num_kv_heads, cw.scale,
                                                cw.block_tables, cw.context_lens, 16, cw.max_context_len, None)
            n_launch = n_sets if n_sets % 2 == 0 or cpg is None else 2 * n_sets
            ms = R.time_rotating([lambda i=i: dec(i) for i in range(n_launch)], reps)
            configs[key] = roof("hbm", cw.algorithmic_bytes(), ms, peaks,
                                {"workload": cw.name, "pool_copies": n_sets,
                                 "includes": "decode + merge launches" +
                                 (", peer stores and barrier" if cpg is not None else "")})
            dec(0)
            torch.cuda.synchronize()
            g_out = (cpg.tensors[0] if cpg is not None else
                     (sharding.gather_heads(o_loc) if world > 1 else o_loc)).clone()
            if cpg is not None:
                cpg.close()
            del cpools
            if key == "cfg5_decode":
                # the AICI fork on this pool: 32 sequences x 4 children, last block each, 4 "layers";
                # eight different sets of 32 parents (and of free blocks) are copied in turn
                rows_ = [cw.block_tables[i, :(c + 15) // 16].tolist() for i, c in enumerate(cw.context_list)]
                used = set(b for r in rows_ for b in r)
                free = [b for b in range(cw.key_cache.shape[0]) if b not in used]
                layers = 4
                kcs = [cw.key_cache] + [cw.key_cache.clone() for _ in range(layers - 1)]
                vcs = [cw.value_cache] + [cw.value_cache.clone() for _ in range(layers - 1)]
                maps = []
                for j in range(8):
                    parents = rows_[(24 * j) % (len(rows_) - 32):][:32]
                    mapping = workloads.fork_block_mapping(parents, 32, 4, free[128 * j:128 * (j + 1)])
                    maps.append((mapping, torch.tensor([x for s_, ds in mapping.items() for d_ in ds
                                                        for x in (s_, d_)], dtype=torch.int64)))
                ms = R.time_rotating([lambda f=f: tch_cuda.copy_blocks(kcs, vcs, f) for _m, f in maps], reps)
                blk_bytes = cw.num_kv_heads * 128 * 16 * 2
                pairs = maps[0][1].numel() // 2
                ok = True
                for s_, ds in maps[0][0].items():
                    for d_ in ds:
                        for l in range(layers):
                            ok = ok and torch.equal(kcs[l][d_].view(torch.int16), kcs[l][s_].view(torch.int16)) \
                                and torch.equal(vcs[l][d_].view(torch.int16), vcs[l][s_].view(torch.int16))
                configs["cfg5_copy_blocks"] = roof(
                    "hbm", pairs * layers * 2 * blk_bytes * 2, ms, peaks,
                    {"workload": "fork of 32 sequences into 4 children, last block each: %d pairs x %d layers"
                                 % (pairs, layers), "bit_exact": R.all_true(ok),
                     "note": "%.0f MB per launch: the written half stays in the write-back L2 during the launch, "
                             "so the fraction of the HBM copy peak can exceed 1" %
                             (pairs * layers * 2 * blk_bytes * 2 / 1e6)})
                del kcs, vcs
            del cw.key_cache, cw.value_cache
            torch.cuda.empty_cache()
            if rank == 0:
                full = make(dev)
                parity[key], _ = decode_parity(full, g_out)
                del full
            torch.cuda.empty_cache()

        # config 5, prefill part (8 chunks of 512) and the cache write of its 4288 tokens
        pw5 = workloads.prefill_mixed_chunks(dev, shard=shard)
        p5_bytes = (pw5.q.numel() * 2 + pw5.k.numel() * 2) * 2
        sets5 = [(pw5.q, pw5.k, pw5.v)] + [(pw5.q.clone(), pw5.k.clone(), pw5.v.clone())
                                           for _ in range(copies_to_stream(p5_bytes, 4 * L2_BYTES) - 1)]
        ms = R.time_rotating([lambda t=t: tch_cuda.flash_attn_varlen(t[0], t[1], t[2], pw5.cu_seqlens_q,
                                                                     pw5.cu_seqlens_k, pw5.max_seqlen_q,
                                                                     pw5.max_seqlen_k, pw5.scale, True)
                              for t in sets5], reps)
        # host cost of one call through the C ABI (argument checks, tensor-map look-up, launch): wall
        # time of back-to-back eager calls on resident inputs, no synchronisation in between
        def host_us(fn, n=200):
            fn()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for _ in range(n):
                fn()
            dt = (time.perf_counter() - t0) / n * 1e6
            torch.cuda.synchronize()
            return dt
        q5, k5, v5 = sets5[0]
        out5 = torch.empty_like(q5)
        import ctypes

        def raw_prefill_call():
            _lib.check("aici_mha_varlen_fwd", _lib.lib().aici_mha_varlen_fwd(
                ctypes.c_void_p(out5.data_ptr()), ctypes.c_void_p(q5.data_ptr()), ctypes.c_void_p(k5.data_ptr()),
                ctypes.c_void_p(v5.data_ptr()), ctypes.c_void_p(pw5.cu_seqlens_q.data_ptr()),
                ctypes.c_void_p(pw5.cu_seqlens_k.data_ptr()), len(pw5.lens_q), q5.shape[0], k5.shape[0], q5.shape[1],
                k5.shape[1], 128, pw5.max_seqlen_q, pw5.max_seqlen_k, *[ctypes.c_int64(x) for x in (
                    q5.stride(0), q5.stride(1), k5.stride(0), k5.stride(1), v5.stride(0), v5.stride(1),
                    out5.stride(0), out5.stride(1))], ctypes.c_float(pw5.scale), 1, 0,
                ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)))
        configs["cfg5_prefill"] = roof("tensor", pw5.flops(), ms, peaks, {
            "workload": pw5.name,
            "host_us_per_call": {"c_abi": host_us(raw_prefill_call),
                                 "python_mirror": host_us(lambda: tch_cuda.flash_attn_varlen(
                                     q5, k5, v5, pw5.cu_seqlens_q, pw5.cu_seqlens_k, pw5.max_seqlen_q,
                                     pw5.max_seqlen_k, pw5.scale, True))}})
        o5 = tch_cuda.flash_attn_varlen(pw5.q, pw5.k, pw5.v, pw5.cu_seqlens_q, pw5.cu_seqlens_k,
                                        pw5.max_seqlen_q, pw5.max_seqlen_k, pw5.scale, True)
        g5 = sharding.gather_heads(o5) if world > 1 else o5
        if rank == 0:
            parity["cfg5_prefill"], _ = prefill_parity(workloads.prefill_mixed_chunks(dev), g5, n_rows=256)
        del sets5
        hkv5 = pw5.k.shape[1]
        n_tok = 4288
        nb5 = n_tok // 16 + 8
        rc_bytes = n_tok * hkv5 * 128 * 2 * 2 * 2
        kk = torch.cat([pw5.k, pw5.k[:n_tok - pw5.k.shape[0]]]).contiguous()
        vv = torch.cat([pw5.v, pw5.v[:n_tok - pw5.v.shape[0]]]).contiguous()
        slots5 = torch.arange(n_tok, dtype=torch.int32, device=dev)
        rc_sets = []
        for j in range(copies_to_stream(rc_bytes, 4 * L2_BYTES)):
            rc_sets.append((kk if j == 0 else kk.clone(), vv if j == 0 else vv.clone(),
                            torch.zeros(nb5, hkv5, 16, 16, 8, dtype=torch.bfloat16, device=dev),
                            torch.zeros(nb5, hkv5, 128, 16, dtype=torch.bfloat16, device=dev)))
        ms = R.time_rotating([lambda t=t: tch_cuda.reshape_and_cache(t[0], t[1], t[2], t[3], slots5)
                              for t in rc_sets], reps)
        ok = True
        if rank == 0:
            from oracle import cpu_oracle as O
            kc5, vc5 = rc_sets[-1][2], rc_sets[-1][3]
            kr, vr = torch.zeros_like(kc5).cpu(), torch.zeros_like(vc5).cpu()
            O.reshape_and_cache(kk.cpu(), vv.cpu(), kr, vr, slots5.cpu())
            ok = torch.equal(kc5.cpu().view(torch.int16), kr.view(torch.int16)) and \
                torch.equal(vc5.cpu().view(torch.int16), vr.view(torch.int16))
        configs["cfg5_reshape_and_cache"] = roof(
            "hbm", rc_bytes, ms, peaks,
            {"workload": "4288 tokens (8 x 512 prefill + 192 decode), block-aligned chunks", "bit_exact": ok,
             "note": "%.0f MB per launch: launch ramp and two memory round trips; the written half stays in "
                     "the write-back L2 during the launch" % (rc_bytes / 1e6)})
        del pw5, rc_sets, kk, vv, o5, g5
        torch.cuda.empty_cache()
        for v_ in configs.values():
            v_["timing"] = "one CUDA graph of back-to-back launches over distinct buffer sets (>= 4x L2 in all), " \
                           "replayed %d times between two events; ms per launch" % reps

    # ---- long-context causal prefill (2 x 32768, 64 q / 8 kv heads; heads split over ranks) ---
    pw = workloads.prefill_long(dev, shard=shard)
    p_steps, p_warm = max(2, min(args.steps, 5)), 3
    hq_p = pw.q.shape[1] * world

    def pstep():
        return tch_cuda.flash_attn_varlen(pw.q, pw.k, pw.v, pw.cu_seqlens_q, pw.cu_seqlens_k,
                                          pw.max_seqlen_q, pw.max_seqlen_k, pw.scale, True)

    pbuf, ppg = None, None
    if fused:
        ppg = sharding.PeerGather(pw.q.shape[0], hq_p, 128, dev, buffers=1)
        ppg.barrier()

        def pstep():  # noqa: F811
            tch_cuda.flash_attn_varlen_peers(ppg.ptrs, hq_p, ppg.head0, pw.q, pw.k, pw.v, pw.cu_seqlens_q,
                                             pw.cu_seqlens_k, pw.max_seqlen_q, pw.max_seqlen_k, pw.scale, True)
            return ppg.tensor
    elif world > 1:
        pbuf = torch.empty(world, pw.q.shape[0], pw.q.shape[1], 128, dtype=torch.bfloat16, device=dev)

    def pgather(o):
        if fused:
            ppg.barrier()
        elif world > 1:
            dist.all_gather_into_tensor(pbuf.view(-1, pbuf.shape[2], 128), o)
    for _ in range(p_warm):
        pgather(pstep())
    R.barrier()
    k_ms = []
    sampler.region("prefill")
    ev0.record()
    for _ in range(p_steps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        o = pstep()
        b.record()
        k_ms.append((a, b))
        pgather(o)
    ev1.record()
    R.barrier()
    p_ms = R.max_over_ranks(ev0.elapsed_time(ev1)) / p_steps
    p_kernel_ms = R.max_over_ranks(sum(a.elapsed_time(b) for a, b in k_ms) / p_steps)
    sampler.region(None)
    sampler.stop()
    clocks = sampler.summary("decode")
    p_flops_local = pw.flops()
    p_tflops = p_flops_local * world / (p_ms * 1e-3) / 1e12
    p_kernel_tflops = p_flops_local / (p_kernel_ms * 1e-3) / 1e12
    status = _lib.last_status()
    if status != 0:
        raise SystemExit("device status word is %d after the prefill region" % status)
    # parity of the gathered prefill output
    if fused:
        p_gathered = o
        local_o = tch_cuda.flash_attn_varlen(pw.q, pw.k, pw.v, pw.cu_seqlens_q, pw.cu_seqlens_k,
                                             pw.max_seqlen_q, pw.max_seqlen_k, pw.scale, True)
        via_nccl = sharding.gather_heads(local_o)
        same = torch.equal(p_gathered.view(torch.int16), via_nccl.contiguous().view(torch.int16))
        parity["prefill_fused_equals_nccl"] = R.all_true(same)
        del local_o, via_nccl
    elif world > 1:
        p_gathered = pbuf.permute(1, 0, 2, 3).reshape(pw.q.shape[0], hq_p, 128)
    else:
        p_gathered = o
    if rank == 0:
        del pw
        torch.cuda.empty_cache()
        parity["prefill"], parity["prefill_rows_checked"] = prefill_parity(workloads.prefill_long(dev), p_gathered)
    bad = []
    for k_, v_ in parity.items():
        if isinstance(v_, list) and (v_[0] > MAX_ABS or v_[1] > MEAN_ABS):
            bad.append("%s max/mean abs error %.3e/%.3e" % (k_, v_[0], v_[1]))
        if k_.endswith("equals_nccl") and v_ is False:
            bad.append(k_ + " is false")
    for k_, v_ in configs.items():
        if v_.get("bit_exact") is False:
            bad.append(k_ + " is not bit-exact")
    parity["bounds"] = {"max_abs": MAX_ABS, "mean_abs": MEAN_ABS}
    parity["ok"] = not bad

    if pg is not None:
        pg.close()
    if ppg is not None:
        ppg.close()
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    cpu_baseline = None
    if world == 1 and not args.no_cpu_baseline:
        cpu_baseline, _, _ = time_cpu(steps=4, warmup=1)

    ratio = DECODE_TRAFFIC_RATIO.get(world)
    config = shared_config(world, step_bytes_local * world)
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": config,
        "run": {
            "launch": ("CUDA-graph replays, %d step%s per graph" % (spg, "" if spg == 1 else "s")) if use_graph else "eager launches",
            "step_call": ("reshape_and_cache, then paged_attention_v1" if args.separate_calls else
                          "aici_decode_step (cache write and decode attention in one call, overlapped)"),
            "pool_copies": n_pools,
            "bytes_streamed_per_gpu_per_step": decode_bytes_local,
            "collective": ("none" if world == 1 else
                           "fused: the decode call stores head outputs into every rank's buffer over NVLink "
                           "(buffers mapped with the library's own peer-memory calls, %s; two used in turn) and "
                           "its last kernel is the ranks' barrier" % (
                               {1: "virtual-memory allocations shared by file descriptor",
                                2: "cudaMalloc blocks shared by CUDA IPC handles"}.get(peer_kind, "?")) if fused else
                           "nccl all_gather of head outputs" +
                           (" (fused gather unavailable: %s)" % fused_fallback if fused_fallback else "")),
        },
        "roofline": {
            "kernel": "paged_decode_kernel (+ the merge launch of the same call)",
            "bound": "hbm", "achieved": achieved_gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
            "frac": achieved_gbs / peaks["hbm_gbs"], "peak_source": peaks["source"],
            "launch_ms": att_ms,
            "traffic": ratio * decode_bytes_local if ratio else None,
            "traffic_note": ("ncu dram read+write of one launch of rank 0's shard at this world size, "
                             "as a ratio to its algorithmic bytes" if ratio else
                             "no ncu capture of this shard size on file"),
        },
        "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": e2e_ms, "host_wall_ms_per_step": e2e_wall_ms,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "note": "q, new k/v, slot map, block tables, context lens copied from one pinned staging "
                        "buffer (one copy) and the gathered output read back every step, in order (copy in, "
                        "kernels, copy out; nothing of one step overlaps the next); the KV cache is "
                        "resident state" + ("; steps alternate between two peer-mapped output buffers, so a "
                                            "peer's next step never writes what this rank still reads"
                                            if fused else "")},
        # this library's kernels inside the timed region, per step: paged_decode (which also writes the
        # step's new tokens to the cache) and paged_merge (whose tail is the cross-GPU barrier when the
        # fused gather is used); with --separate-calls reshape_and_cache is a third launch
        "gpu_launches": (3 if args.separate_calls else 2) * args.steps,
        "clocks": clocks,
        "parity": parity,
        "configs": configs,
        "prefill": {
            "workload": "prefill_2x32768_gqa64-8_causal_d128", "tflops": p_tflops, "ms_per_step": p_ms,
            "steps": p_steps, "flops_per_step": p_flops_local * world,
            "roofline": {"kernel": "varlen_prefill_kernel", "bound": "tensor", "achieved": p_kernel_tflops,
                         "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s",
                         "frac": p_kernel_tflops / peaks["bf16_tflops_sustained"],
                         "frac_of_burst_peak": p_kernel_tflops / peaks["bf16_tflops"],
                         "peak_source": peaks["source"] + " (sustained cuBLAS bf16)", "launch_ms": p_kernel_ms,
                         "traffic": PREFILL_TRAFFIC_BYTES.get(world),
                         "traffic_note": ("ncu dram read+write of this launch (one-pass capture of `--profile "
                                          "prefill_full`); q, k, v and output are 2.42 GB, the rest is K/V "
                                          "fetched again by later row tiles (268 MB of K/V against a 126 MB L2), "
                                          "9 % of the HBM rate" if world in PREFILL_TRAFFIC_BYTES else
                                          "not captured at this world size")},
            "clocks": sampler.summary("prefill"),
        },
    }
    if cpu_baseline is not None:
        line["cpu_baseline"] = cpu_baseline
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    if bad:
        raise SystemExit("parity check failed: " + "; ".join(bad))


# ---------------------------------------------------------------------------------------------
# --suite: device timings of all five configurations at the current world size (no oracle here;
# parity at every GPU count is covered by tests/test_gpu_multi.py)
# ---------------------------------------------------------------------------------------------
def run_suite(args):
    import torch.distributed as dist
    from aici_b200 import tch_cuda, _lib
    import workloads

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    peaks = load_peaks()
    shard = workloads.Shard(rank=rank, world=world)
    flush = torch.empty(512 << 20, dtype=torch.uint8, device=dev)  # 4x the L2
    iters, warm = max(5, min(args.steps, 20)), 3
    rows = []

    def reduce_max(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timed(fn, gather_fn=None):
        """median device time of fn over `iters` launches, L2 flushed before each; max over ranks"""
        ks, gs = [], []
        for i in range(warm + iters):
            if world > 1:
                dist.barrier()
            flush.zero_()  # also gives the host time to queue the launches behind it
            a, b, c = (torch.cuda.Event(enable_timing=True) for _ in range(3))
            a.record()
            o = fn()
            b.record()
            if gather_fn is not None and world > 1:
                gather_fn(o)
            c.record()
            torch.cuda.synchronize()
            if i >= warm:
                ks.append(a.elapsed_time(b))
                gs.append(b.elapsed_time(c))
        return reduce_max(statistics.median(ks)), reduce_max(statistics.median(gs))

    def add(name, kind, work_local, k_ms, g_ms, extra=None):
        total = work_local * world
        if kind == "hbm":
            ach = work_local / (k_ms * 1e-3) / 1e9
            peak, unit = peaks["hbm_gbs"], "GB/s"
        elif kind == "pcie":  # host <-> device traffic: no measured peak on file, fraction omitted
            ach = work_local / (k_ms * 1e-3) / 1e9
            peak, unit = None, "GB/s"
        else:
            ach = work_local / (k_ms * 1e-3) / 1e12
            peak, unit = peaks["bf16_tflops_sustained"], "TFLOP/s"
        row = {"config": name, "n_gpus": world, "kernel_ms": k_ms, "gather_ms": g_ms,
               "work_per_gpu": work_local, "work_total": total, "achieved_per_gpu": ach, "unit": unit,
               "frac_of_peak": (ach / peak if peak else None), "aggregate": ach * world,
               "aggregate_with_gather": work_local * world / ((k_ms + g_ms) * 1e-3) / (1e9 if kind == "hbm" else 1e12)}
        if extra:
            row.update(extra)
        rows.append(row)

    def gather_into(buf):
        def g(o):
            dist.all_gather_into_tensor(buf.view(-1, o.shape[1], 128), o)
        return g

    # config 1: small varlen prefill
    pw = workloads.prefill_small(dev, shard=shard)
    buf = torch.empty(world, *pw.q.shape, dtype=torch.bfloat16, device=dev)
    k_ms, g_ms = timed(lambda: tch_cuda.flash_attn_varlen(pw.q, pw.k, pw.v, pw.cu_seqlens_q, pw.cu_seqlens_k,
                                                          pw.max_seqlen_q, pw.max_seqlen_k, pw.scale, True),
                       gather_into(buf))
    add("1 " + pw.name, "tensor", pw.flops(), k_ms, g_ms)
    del pw, buf

    # configs 2, 3, 5(decode)
    for label, make in (("2", workloads.decode_llama2_7b), ("3", workloads.decode_llama3_8b),
                        ("5-decode", workloads.decode_mixed_step)):
        w = make(dev, shard=shard)
        out = torch.empty_like(w.query)
        buf = torch.empty(world, *w.query.shape, dtype=torch.bfloat16, device=dev)

        def dec(w=w, out=out):
            tch_cuda.paged_attention_v1(out, w.query, w.key_cache, w.value_cache, w.num_kv_heads, w.scale,
                                        w.block_tables, w.context_lens, 16, w.max_context_len, None)
            return out
        k_ms, g_ms = timed(dec, gather_into(buf))
        r_ms, _ = timed(lambda w=w: tch_cuda.reshape_and_cache(w.new_key, w.new_value, w.key_cache,
                                                               w.value_cache, w.slot_mapping))
        add(label + " " + w.name, "hbm", w.algorithmic_bytes(), k_ms, g_ms,
            {"reshape_and_cache_ms": r_ms, "max_context_len": w.max_context_len})
        if label == "5-decode":
            # fork copy, bandwidth variant: every block of the first 8 sequences to 4 children
            used = set(w.block_tables.cpu().flatten().tolist())
            free = [b for b in range(w.key_cache.shape[0]) if b not in used]
            rows_ = [w.block_tables[i, :(c + 15) // 16].tolist() for i, c in enumerate(w.context_list)]
            mapping = workloads.fork_block_mapping(rows_, 8, 4, free, whole_sequence=True)
            pairs = sum(len(v) for v in mapping.values())
            flat = torch.tensor([x for s_, ds in mapping.items() for d_ in ds for x in (s_, d_)], dtype=torch.int64)
            c_ms, _ = timed(lambda: tch_cuda.copy_blocks([w.key_cache], [w.value_cache], flat))
            blk_bytes = w.num_kv_heads * 128 * 16 * 2
            add("5-copy_blocks whole-sequence fork (%d pairs, 1 layer)" % pairs, "hbm",
                pairs * 2 * blk_bytes * 2, c_ms, 0.0)
            last = workloads.fork_block_mapping(rows_, 32, 4, free)
            c2_ms, _ = timed(lambda: tch_cuda.copy_blocks([w.key_cache] * 4, [w.value_cache] * 4, last))
            add("5-copy_blocks last-block fork (128 pairs, 4 layers)", "hbm", 128 * 4 * 2 * blk_bytes * 2, c2_ms, 0.0)
        del w, out, buf
        torch.cuda.empty_cache()

    # config 5 prefill part and its cache write (4288 tokens)
    pw = workloads.prefill_mixed_chunks(dev, shard=shard)
    buf = torch.empty(world, *pw.q.shape, dtype=torch.bfloat16, device=dev)
    k_ms, g_ms = timed(lambda: tch_cuda.flash_attn_varlen(pw.q, pw.k, pw.v, pw.cu_seqlens_q, pw.cu_seqlens_k,
                                                          pw.max_seqlen_q, pw.max_seqlen_k, pw.scale, True),
                       gather_into(buf))
    add("5-prefill " + pw.name, "tensor", pw.flops(), k_ms, g_ms)
    hkv = pw.k.shape[1]
    kc = torch.zeros(4288 // 16 + 8, hkv, 16, 16, 8, dtype=torch.bfloat16, device=dev)
    vc = torch.zeros(4288 // 16 + 8, hkv, 128, 16, dtype=torch.bfloat16, device=dev)
    kk = torch.cat([pw.k, pw.k[:192]]).contiguous()
    slots = torch.arange(4288, dtype=torch.int32, device=dev) + 5
    r_ms, _ = timed(lambda: tch_cuda.reshape_and_cache(kk, kk, kc, vc, slots))
    add("5-reshape_and_cache 4288 tokens, chunks starting mid-block", "hbm", 4288 * hkv * 128 * 2 * 2 * 2, r_ms, 0.0)
    slots_a = torch.arange(4288, dtype=torch.int32, device=dev)
    r_ms, _ = timed(lambda: tch_cuda.reshape_and_cache(kk, kk, kc, vc, slots_a))
    add("5-reshape_and_cache 4288 tokens, block-aligned chunks", "hbm", 4288 * hkv * 128 * 2 * 2 * 2, r_ms, 0.0)
    del pw, buf, kc, vc, kk

    # prefill from the paged cache (the "next" row): the same long-context problem with K/V living
    # in cache blocks, against gather_cached_kv + packed prefill (what rLLM's call sequence does)
    L = 8192
    pw = workloads.prefill_long(dev, shard=shard, seqlen=L)
    hkv = pw.k.shape[1]
    nblk = 2 * L // 16 + 8
    table, rows_ = workloads.build_block_tables([L, L], nblk, 4100)
    slots = torch.tensor([r[t // 16] * 16 + t % 16 for r in rows_ for t in range(L)], dtype=torch.int32, device=dev)
    kc = torch.zeros(nblk, hkv, 16, 16, 8, dtype=torch.bfloat16, device=dev)
    vc = torch.zeros(nblk, hkv, 128, 16, dtype=torch.bfloat16, device=dev)
    tch_cuda.reshape_and_cache(pw.k, pw.v, kc, vc, slots)
    table_d = table.to(dev)
    cl = torch.tensor([L, L], dtype=torch.int32, device=dev)
    kg, vg = torch.empty_like(pw.k), torch.empty_like(pw.v)

    def gather_then_packed():
        tch_cuda.gather_cached_kv(kg, vg, kc, vc, slots)
        return tch_cuda.flash_attn_varlen(pw.q, kg, vg, pw.cu_seqlens_q, pw.cu_seqlens_k, L, L, pw.scale, True)
    k_ms, _ = timed(gather_then_packed)
    add("next: gather_cached_kv + packed prefill 2x%d" % L, "tensor", pw.flops(), k_ms, 0.0)
    k_ms, _ = timed(lambda: tch_cuda.flash_attn_varlen_paged(pw.q, kc, vc, pw.cu_seqlens_q, cl, table_d, L, L,
                                                             pw.scale, True))
    add("next: paged prefill 2x%d (K/V read through block tables)" % L, "tensor", pw.flops(), k_ms, 0.0)
    del pw, kc, vc, kg, vg

    # swap_blocks (the "next" row): 1024 blocks of one layer's K cache out to page-locked host memory
    # and back in, one launch each, against one cudaMemcpyAsync per block (the reference's way)
    hkv = max(1, 8 // world)
    nblk = 2048
    kc = torch.randn(nblk, hkv, 16, 16, 8, device=dev).to(torch.bfloat16)
    host = torch.empty(nblk, hkv, 16, 16, 8, dtype=torch.bfloat16).pin_memory()
    gsel = torch.randperm(nblk)[:1024]
    hsel = torch.randperm(nblk)[:1024]
    out_pairs = torch.stack([gsel, hsel], 1).reshape(-1).to(torch.int64)
    in_pairs = torch.stack([hsel, gsel], 1).reshape(-1).to(torch.int64)
    blk_bytes = hkv * 128 * 16 * 2
    o_ms, _ = timed(lambda: tch_cuda.swap_blocks(kc, host, out_pairs))
    add("next: swap_blocks out, 1024 blocks of %d KB to page-locked host" % (blk_bytes >> 10), "pcie",
        1024 * blk_bytes, o_ms, 0.0)
    i_ms, _ = timed(lambda: tch_cuda.swap_blocks(host, kc, in_pairs))
    add("next: swap_blocks in, 1024 blocks of %d KB from page-locked host" % (blk_bytes >> 10), "pcie",
        1024 * blk_bytes, i_ms, 0.0)

    def per_block_copies():
        for s_, d_ in zip(gsel.tolist(), hsel.tolist()):
            host[d_].copy_(kc[s_], non_blocking=True)
    m_ms, _ = timed(per_block_copies)
    add("next: (comparison) one async copy per block, same 1024 blocks out", "pcie", 1024 * blk_bytes, m_ms, 0.0)
    del kc, host

    # BatchInfo staging (the "next" row): config 3's decode step (256 sequences) described as
    # entries, built natively into one page-locked buffer and uploaded with one copy; host wall time
    from aici_b200 import batch_info
    w = workloads.decode_llama3_8b(dev, shard=shard)
    tables = w.block_tables.cpu()
    offs = torch.arange(16, dtype=torch.int64)
    ent = []
    for i, c in enumerate(w.context_list):
        blocks = tables[i, :(c + 15) // 16].to(torch.int64)
        ent.append((i, torch.tensor([7], dtype=torch.int32), (blocks[:, None] * 16 + offs[None, :]).reshape(-1)[:c].contiguous()))
    bld = batch_info.BatchInfoBuilder(block_size=16, max_model_len=1 << 20, device=dev, gather_mapping=False)
    walls = []
    for it in range(warm + iters):
        for sid, tok, sl in ent:
            bld.add_arrays(sid, tok, sl)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        bi = bld.finish(it)
        torch.cuda.synchronize()
        walls.append((time.perf_counter() - t0) * 1e3)
    assert torch.equal(bi.paged_context_lens, w.context_lens)
    rows.append({"config": "next: BatchInfo build + one upload, config 3 decode step (256 sequences)",
                 "n_gpus": world, "host_wall_ms": statistics.median(walls[warm:]),
                 "bytes_uploaded": int(bi.layout.total_bytes), "uploads": 1})
    del w, bld, bi, ent

    # config 4: long prefill
    pw = workloads.prefill_long(dev, shard=shard)
    buf = torch.empty(world, *pw.q.shape, dtype=torch.bfloat16, device=dev)
    k_ms, g_ms = timed(lambda: tch_cuda.flash_attn_varlen(pw.q, pw.k, pw.v, pw.cu_seqlens_q, pw.cu_seqlens_k,
                                                          pw.max_seqlen_q, pw.max_seqlen_k, pw.scale, True),
                       gather_into(buf))
    add("4 " + pw.name, "tensor", pw.flops(), k_ms, g_ms, {"frac_of_burst_peak": pw.flops() / (k_ms * 1e-3) / 1e12 / peaks["bf16_tflops"]})
    status = _lib.last_status()
    if rank == 0:
        print(json.dumps({"suite": rows, "n_gpus": world, "status": status, "peaks": peaks,
                          "timing": "median of %d launches, 512 MB L2 flush before each, CUDA events, max over ranks" % iters}))
    if world > 1:
        dist.destroy_process_group()

def run_profile_case(args):
    """Small single-GPU cases for profiler captures (at most a few GB on the device, three launches):
    the numbers printed here are not benchmark values.  `decode` with --profile-world N runs rank 0's
    kv-head shard of an N-GPU run (all 64 sequences, 32 / N heads) -- the launch the scaling run
    times at that N; without it, a 16-sequence case of the one-GPU shape."""
    from aici_b200 import tch_cuda
    import workloads
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    if args.profile == "decode":
        if args.profile_world > 1:
            w = workloads.decode_llama2_7b(dev, shard=workloads.Shard(0, args.profile_world))
        else:
            w = workloads.decode_llama2_7b(dev, num_seqs=16, pool_blocks=4096)
        out = torch.empty_like(w.query)
        for _ in range(3):
            tch_cuda.reshape_and_cache(w.new_key, w.new_value, w.key_cache, w.value_cache, w.slot_mapping)
            tch_cuda.paged_attention_v1(out, w.query, w.key_cache, w.value_cache, w.num_kv_heads, w.scale,
                                        w.block_tables, w.context_lens, 16, w.max_context_len, None)
        torch.cuda.synchronize()
        print(json.dumps({"profile_case": "decode", "seqs": w.query.shape[0], "heads": w.num_heads,
                          "algorithmic_bytes": w.algorithmic_bytes()}))
    elif args.profile == "small_ops":
        # the short launches of the mixed step, each three times with the L2 flushed before it:
        # cache write of 4288 tokens, fork copy of 128 pairs x 4 layers, prefill of 8 x 512
        pw = workloads.prefill_mixed_chunks(dev)
        flush = torch.empty(4 * L2_BYTES, dtype=torch.uint8, device=dev)
        n_tok, hkv = 4288, pw.k.shape[1]
        kk = torch.cat([pw.k, pw.k[:n_tok - pw.k.shape[0]]]).contiguous()
        kc = torch.zeros(n_tok // 16 + 8, hkv, 16, 16, 8, dtype=torch.bfloat16, device=dev)
        vc = torch.zeros(n_tok // 16 + 8, hkv, 128, 16, dtype=torch.bfloat16, device=dev)
        slots = torch.arange(n_tok, dtype=torch.int32, device=dev)
        pool_k = [torch.zeros(1024, hkv, 16, 16, 8, dtype=torch.bfloat16, device=dev) for _ in range(4)]
        pool_v = [torch.zeros(1024, hkv, 128, 16, dtype=torch.bfloat16, device=dev) for _ in range(4)]
        pairs = torch.tensor([x for i in range(128) for x in (i, 512 + i)], dtype=torch.int64)
        for _ in range(3):
            flush.zero_()
            tch_cuda.reshape_and_cache(kk, kk, kc, vc, slots)
            flush.zero_()
            tch_cuda.copy_blocks(pool_k, pool_v, pairs)
            flush.zero_()
            tch_cuda.flash_attn_varlen(pw.q, pw.k, pw.v, pw.cu_seqlens_q, pw.cu_seqlens_k, pw.max_seqlen_q,
                                       pw.max_seqlen_k, pw.scale, True)
        torch.cuda.synchronize()
        print(json.dumps({"profile_case": "small_ops", "reshape_and_cache_bytes": n_tok * hkv * 128 * 8,
                          "copy_blocks_bytes": 128 * 4 * 2 * hkv * 128 * 16 * 2 * 2, "prefill_flops": pw.flops()}))
    elif args.profile == "prefill_chunks":
        pw = workloads.prefill_mixed_chunks(dev)
        flush = torch.empty(4 * L2_BYTES, dtype=torch.uint8, device=dev)
        for _ in range(3):
            flush.zero_()
            tch_cuda.flash_attn_varlen(pw.q, pw.k, pw.v, pw.cu_seqlens_q, pw.cu_seqlens_k, pw.max_seqlen_q,
                                       pw.max_seqlen_k, pw.scale, True)
        torch.cuda.synchronize()
        print(json.dumps({"profile_case": "prefill_chunks", "flops": pw.flops()}))
    else:
        # prefill_full: the benchmark's own 2 x 32768 launch (2.4 GB on the device, 33 ms), twice; only
        # for captures that take one pass (DRAM byte counters), so that nothing is saved or restored
        seqlen, reps = (32768, 2) if args.profile == "prefill_full" else (4096, 3)
        pw = workloads.prefill_long(dev, seqlen=seqlen)
        for _ in range(reps):
            tch_cuda.flash_attn_varlen(pw.q, pw.k, pw.v, pw.cu_seqlens_q, pw.cu_seqlens_k, pw.max_seqlen_q,
                                       pw.max_seqlen_k, pw.scale, True)
        torch.cuda.synchronize()
        io = sum(t.numel() * t.element_size() for t in (pw.q, pw.k, pw.v)) + pw.q.numel() * pw.q.element_size()
        print(json.dumps({"profile_case": args.profile, "seqlen": seqlen, "flops": pw.flops(),
                          "q_k_v_out_bytes": io}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="launch the decode step eagerly instead of replaying a CUDA graph")
    ap.add_argument("--steps-per-graph", type=int, default=0,
                    help="timed decode steps held by one CUDA graph (0: one turn through the pool copies and "
                         "output buffers, at least 4; 1: one graph replay per step)")
    ap.add_argument("--gather", default="fused", choices=["fused", "nccl"],
                    help="multi-GPU head-output gather: fused into the attention epilogue (default) or NCCL")
    ap.add_argument("--separate-calls", action="store_true",
                    help="make the decode step as two library calls (reshape_and_cache, paged_attention_v1) "
                         "instead of the fused aici_decode_step")
    ap.add_argument("--headline-only", action="store_true",
                    help="skip the per-configuration entries (configs 3 and 5) of the JSON line")
    ap.add_argument("--profile-step", type=int, default=None,
                    help="bracket this step of the timed region with cudaProfilerStart/Stop "
                         "(what rLLM's --profile-step does), for captures limited to the profiler API range")
    ap.add_argument("--suite", action="store_true",
                    help="time all five configurations at the current world size and print one JSON object")
    ap.add_argument("--profile", default=None, choices=["decode", "prefill", "prefill_full", "prefill_chunks", "small_ops"],
                    help="run a small case three times for a profiler capture and exit")
    ap.add_argument("--profile-world", type=int, default=1,
                    help="with --profile decode: run rank 0's shard of a run on this many GPUs")
    args = ap.parse_args()
    if args.profile:
        run_profile_case(args)
        return
    if args.suite:
        run_suite(args)
        return
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
