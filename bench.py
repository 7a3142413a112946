#!/usr/bin/env python
"""Benchmark of the attention hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one decode step of the Llama-2-7B-shaped paged workload (batch 64, 32 MHA heads,
head size 128, block size 16, contexts uniform in [512, 4096], 16384-block pool): the cache
write of the 64 new tokens (reshape_and_cache) followed by decode attention over the paged
cache (paged_attention_v1).  With N > 1 the KV heads are split over the ranks (tensor-parallel
layout) and the head outputs are all-gathered over NCCL inside the step, so the total work is
fixed ("strong" scaling).  The metric is the achieved HBM traffic rate in TB/s computed from
the ALGORITHMIC bytes of the step (K and V once per (sequence, kv head), q, out, block tables,
context lengths, and the cache write), aggregated over all ranks.

The line also carries the long-context causal prefill throughput (2 x 32768 tokens, 64 q / 8 kv
heads) in TFLOP/s under "prefill", the roofline of the dominant decode kernel, an end-to-end
figure through the public API with host buffers, and the CPU baseline: the PyTorch-CPU port of
rLLM's own CPU kernels timed on a bounded sample of the same workload.

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
CPU_SAMPLE_SEQS = 8
# DRAM bytes (read + write) of paged_decode_kernel per algorithmic byte, from an ncu capture of
# the 16-sequence case that `--profile decode` runs; traffic grows in proportion to the tokens
# read, so the ratio carries over to the full launch.
DECODE_TRAFFIC_RATIO = 1.011


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML (read-only) while a region runs."""

    def __init__(self, index, period=0.02):
        super().__init__(daemon=True)
        self.index, self.period = index, period
        self.samples, self.reasons, self.max_mhz = [], set(), None
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
                r = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self.period)

    def stop(self):
        self._stop_evt.set()
        if self.is_alive():
            self.join(timeout=2)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}
        return {"sm_mhz": int(statistics.median(self.samples)), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def physical_gpu_index(local_rank):
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except Exception:
            return local_rank
    return local_rank


# ---------------------------------------------------------------------------------------------
# CPU arm: the PyTorch-CPU port of rLLM's CPU kernels on a bounded sample of the workload
# ---------------------------------------------------------------------------------------------
def cpu_sample_inputs(n_seqs):
    """The first n_seqs sequences of the decode workload with their blocks compacted into a small
    fp32 pool (the CPU build of rLLM runs fp32).  Contexts and tables are the benchmark's own."""
    from aici_b200 import workloads
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
                slots=slots, hkv=hkv, bytes=kv + qo + bt + cw)


def cpu_step(c):
    from oracle import refkernels_cpu as R
    R.reshape_and_cache(c["nk"], c["nv"], c["kc"], c["vc"], c["slots"])
    return R.decode_step_cpu(c["q"], c["kc"], c["vc"], c["hkv"], 1.0 / 128 ** 0.5, c["table"], c["ctx"], 16)


def time_cpu(steps, warmup):
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    c = cpu_sample_inputs(CPU_SAMPLE_SEQS)
    for _ in range(warmup):
        cpu_step(c)
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_step(c)
    dt = (time.perf_counter() - t0) / max(steps, 1)
    return {"value": c["bytes"] / dt / 1e12, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": "first %d of the 64 sequences (%.1f MB algorithmic), fp32, gather_cached_kv + "
                      "repeat_kv + per-sequence scaled_dot_product_attention as in refkernels.rs, "
                      "%.3f s per step" % (CPU_SAMPLE_SEQS, c["bytes"] / 1e6, dt)}, dt


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps, warm = max(1, args.steps), max(1, args.warmup)
    cb, dt = time_cpu(steps, warm)
    line = {
        "impl": "reference", "metric": METRIC, "value": cb["value"], "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": warm, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "note": "CPU path of the reference (refkernels.rs port), bounded sample"},
        "cpu_baseline": cb,
        "e2e": {"value": cb["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------
def run_ours(args):
    import torch.distributed as dist
    from aici_b200 import tch_cuda, workloads, _lib

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node %d" % args.gpus)
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    peaks = load_peaks()
    shard = workloads.Shard(rank=rank, world=world)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- decode workload ------------------------------------------------------------------
    w = workloads.decode_llama2_7b(dev, shard=shard)
    S, hq_local = w.query.shape[0], w.query.shape[1]
    out = torch.empty_like(w.query)
    gathered = torch.empty(world, S, hq_local, 128, dtype=torch.bfloat16, device=dev) if world > 1 else None
    step_bytes_local = w.algorithmic_bytes() + w.cache_write_bytes()
    decode_bytes_local = w.algorithmic_bytes()
    fused = world > 1 and args.gather == "fused"
    pg = None
    fused_fallback = None
    if fused:
        from aici_b200 import sharding
        # peer-mapped buffers come from torch's symmetric-memory allocator; if any rank cannot set
        # them up, every rank falls back to the NCCL gather (and the JSON line says so)
        try:
            pg = sharding.PeerGather(S, hq_local * world, 128, dev)
            ok = 1
        except Exception as e:  # noqa: BLE001
            fused_fallback, ok = "%s: %s" % (type(e).__name__, str(e)[:120]), 0
        flag = torch.tensor([ok], dtype=torch.int32, device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag.item()) == 0:
            fused, pg = False, None
            fused_fallback = fused_fallback or "another rank could not map peer memory"
        else:
            pg.barrier()

    def attention(q, bt, cl):
        """decode attention + head gather: fused epilogue (peer stores + barrier) or NCCL all-gather"""
        if fused:
            tch_cuda.paged_attention_v1_peers(pg.ptrs, hq_local * world, pg.head0, q, w.key_cache, w.value_cache,
                                              w.num_kv_heads, w.scale, bt, cl, 16, w.max_context_len)
            pg.barrier()
            return pg.tensor
        tch_cuda.paged_attention_v1(out, q, w.key_cache, w.value_cache, w.num_kv_heads, w.scale, bt, cl, 16,
                                    w.max_context_len, None)
        if world > 1:
            dist.all_gather_into_tensor(gathered.view(-1, hq_local, 128), out)
            return gathered
        return out

    def step():
        tch_cuda.reshape_and_cache(w.new_key, w.new_value, w.key_cache, w.value_cache, w.slot_mapping)
        attention(w.query, w.block_tables, w.context_lens)

    sampler = ClockSampler(physical_gpu_index(local_rank))
    sampler.start()
    for _ in range(args.warmup):
        step()
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    # The step (cache write, decode, merge, cross-GPU barrier) is a handful of short launches, so
    # it is captured once into a CUDA graph and replayed; the NCCL variant is launched eagerly.
    use_graph = (world == 1 or fused) and not args.no_graph
    if use_graph:
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            step()  # sizes this stream's workspace outside the capture
        torch.cuda.current_stream(dev).wait_stream(side)
        barrier()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            step()
        for _ in range(3):
            graph.replay()
        barrier()
        ev0.record()
        for _ in range(args.steps):
            graph.replay()
        ev1.record()
        barrier()
    else:
        ev0.record()
        for _ in range(args.steps):
            step()
        ev1.record()
        barrier()
    # The decode call alone (decode + merge launches; with the fused gather their stores to the
    # peers), for the roofline: K back-to-back replays of a graph holding just that call, so the
    # figure is device time and does not depend on how fast the host can launch (eager launches
    # with per-step events when graphs are off).
    def attention_only():
        if fused:
            tch_cuda.paged_attention_v1_peers(pg.ptrs, hq_local * world, pg.head0, w.query, w.key_cache,
                                              w.value_cache, w.num_kv_heads, w.scale, w.block_tables,
                                              w.context_lens, 16, w.max_context_len)
        else:
            tch_cuda.paged_attention_v1(out, w.query, w.key_cache, w.value_cache, w.num_kv_heads, w.scale,
                                        w.block_tables, w.context_lens, 16, w.max_context_len, None)

    if use_graph:
        side.wait_stream(torch.cuda.current_stream(dev))
        att_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(att_graph, stream=side):
            attention_only()
        for _ in range(3):
            att_graph.replay()
        barrier()
        ea, eb = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ea.record()
        for _ in range(args.steps):
            att_graph.replay()
        eb.record()
        barrier()
        att_local_ms = ea.elapsed_time(eb) / args.steps
    else:
        att_ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                  for _ in range(args.steps)]
        for i in range(args.steps):
            tch_cuda.reshape_and_cache(w.new_key, w.new_value, w.key_cache, w.value_cache, w.slot_mapping)
            att_ev[i][0].record()
            attention_only()
            att_ev[i][1].record()
            if fused:
                pg.barrier()
            elif world > 1:
                dist.all_gather_into_tensor(gathered.view(-1, hq_local, 128), out)
        barrier()
        att_local_ms = sum(a.elapsed_time(b) for a, b in att_ev) / args.steps
    barrier()
    ms_total = max_over_ranks(ev0.elapsed_time(ev1))
    ms_step = ms_total / args.steps
    att_ms = max_over_ranks(att_local_ms)
    status = _lib.last_status()
    if status != 0:
        raise SystemExit("device status word is %d after the timed region" % status)
    value = step_bytes_local * world / (ms_step * 1e-3) / 1e12
    achieved_gbs = decode_bytes_local / (att_ms * 1e-3) / 1e9

    # ---- end to end through the public API with host buffers -------------------------------
    # The step's inputs (q, new k/v, slot map, block tables, context lens) sit in ONE page-locked
    # staging buffer at 256-byte aligned offsets and reach the device with ONE copy per step into a
    # buffer of the same layout; the kernels read views of it.
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
    host_out = torch.empty((S, hq_local * world, 128) if world > 1 else out.shape, dtype=out.dtype).pin_memory()
    h2d = sum(t.numel() * t.element_size() for t in parts.values())
    d2h = host_out.numel() * host_out.element_size()

    def e2e_step():
        dev_in.copy_(staging, non_blocking=True)
        tch_cuda.reshape_and_cache(d["nk"], d["nv"], w.key_cache, w.value_cache, d["slots"])
        o = attention(d["q"], d["bt"], d["cl"])
        if world > 1 and not fused:
            o = o.permute(1, 0, 2, 3).reshape(S, hq_local * world, 128)
        host_out.copy_(o, non_blocking=True)

    for _ in range(max(3, args.warmup // 2)):
        e2e_step()
    barrier()
    e2e_run = e2e_step
    if use_graph:
        # the whole step -- the copy in, the kernels, the copy out -- as one graph replay
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            e2e_step()
        torch.cuda.current_stream(dev).wait_stream(side)
        barrier()
        e2e_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(e2e_graph, stream=side):
            e2e_step()
        e2e_run = e2e_graph.replay
        for _ in range(3):
            e2e_run()
        barrier()
    t0 = time.perf_counter()
    ev0.record()
    for _ in range(args.steps):
        e2e_run()
    ev1.record()
    barrier()
    e2e_ms = max_over_ranks(max(ev0.elapsed_time(ev1), (time.perf_counter() - t0) * 1e3)) / args.steps
    e2e_value = step_bytes_local * world / (e2e_ms * 1e-3) / 1e12

    # ---- long-context causal prefill (2 x 32768, 64 q / 8 kv heads; heads split over ranks) ---
    del w.key_cache, w.value_cache
    torch.cuda.empty_cache()
    pw = workloads.prefill_long(dev, shard=shard)
    p_steps, p_warm = max(2, min(args.steps, 5)), 3

    def pstep():
        return tch_cuda.flash_attn_varlen(pw.q, pw.k, pw.v, pw.cu_seqlens_q, pw.cu_seqlens_k,
                                          pw.max_seqlen_q, pw.max_seqlen_k, pw.scale, True)

    pbuf, ppg = None, None
    if fused:
        ppg = sharding.PeerGather(pw.q.shape[0], pw.q.shape[1] * world, 128, dev)
        ppg.barrier()

        def pstep():  # noqa: F811
            tch_cuda.flash_attn_varlen_peers(ppg.ptrs, pw.q.shape[1] * world, ppg.head0, pw.q, pw.k, pw.v,
                                             pw.cu_seqlens_q, pw.cu_seqlens_k, pw.max_seqlen_q,
                                             pw.max_seqlen_k, pw.scale, True)
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
    barrier()
    k_ms = []
    ev0.record()
    for _ in range(p_steps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        o = pstep()
        b.record()
        k_ms.append((a, b))
        pgather(o)
    ev1.record()
    barrier()
    p_ms = max_over_ranks(ev0.elapsed_time(ev1)) / p_steps
    p_kernel_ms = max_over_ranks(sum(a.elapsed_time(b) for a, b in k_ms) / p_steps)
    clocks = sampler.stop()
    p_flops_local = pw.flops()
    p_tflops = p_flops_local * world / (p_ms * 1e-3) / 1e12
    p_kernel_tflops = p_flops_local / (p_kernel_ms * 1e-3) / 1e12
    status = _lib.last_status()
    if status != 0:
        raise SystemExit("device status word is %d after the prefill region" % status)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    cpu_baseline = None
    if world == 1 and not args.no_cpu_baseline:
        cpu_baseline, _ = time_cpu(steps=8, warmup=1)

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {
            "workload": WORKLOAD, "sharding": "kv-heads/%d" % world,
            "l2": "no flush: each step streams %.2f GB of K/V per GPU, far above the 126 MB L2" % (
                decode_bytes_local / 1e9),
            "algorithmic_bytes_per_step": step_bytes_local * world,
            "launch": "one CUDA-graph replay per step" if use_graph else "eager launches",
            "collective": ("none" if world == 1 else
                           "fused: attention epilogue stores head outputs into every rank's buffer over "
                           "NVLink (peer-mapped symmetric memory), then a signal barrier" if fused else
                           "nccl all_gather of head outputs" +
                           (" (fused gather unavailable: %s)" % fused_fallback if fused_fallback else "")),
        },
        "roofline": {
            "kernel": "paged_decode_kernel (+ plan and merge launches of the same call)",
            "bound": "hbm", "achieved": achieved_gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
            "frac": achieved_gbs / peaks["hbm_gbs"], "peak_source": peaks["source"],
            "launch_ms": att_ms,
            "traffic": DECODE_TRAFFIC_RATIO * decode_bytes_local,
            "traffic_note": "ncu dram read+write of a 16-sequence launch, scaled by bytes",
        },
        "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": e2e_ms, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h,
                "note": "q, new k/v, slot map, block tables, context lens copied from one pinned staging "
                        "buffer (one copy) and the output read back every step; the KV cache is resident state"},
        # this library's kernels inside the timed region, per step: reshape_and_cache, paged_decode,
        # paged_merge, and the cross-GPU barrier kernel when the fused gather is used
        "gpu_launches": (4 if fused else 3) * args.steps,
        "clocks": clocks,
        "prefill": {
            "workload": pw.name + "_causal_d128", "tflops": p_tflops, "ms_per_step": p_ms, "steps": p_steps,
            "flops_per_step": p_flops_local * world,
            "roofline": {"kernel": "varlen_prefill_kernel", "bound": "tensor", "achieved": p_kernel_tflops,
                         "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s",
                         "frac": p_kernel_tflops / peaks["bf16_tflops_sustained"],
                         "frac_of_burst_peak": p_kernel_tflops / peaks["bf16_tflops"],
                         "peak_source": peaks["source"] + " (sustained cuBLAS bf16)", "launch_ms": p_kernel_ms,
                         "traffic": None},
        },
    }
    if cpu_baseline is not None:
        line["cpu_baseline"] = cpu_baseline
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()



# ---------------------------------------------------------------------------------------------
# --suite: device timings of all five configurations at the current world size (no oracle here;
# parity at every GPU count is covered by tests/test_gpu_multi.py)
# ---------------------------------------------------------------------------------------------
def run_suite(args):
    import torch.distributed as dist
    from aici_b200 import tch_cuda, workloads, _lib

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
    """Small single-GPU cases for profiler captures (a few hundred MB, three launches): the
    numbers printed here are not benchmark values."""
    from aici_b200 import tch_cuda, workloads
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    if args.profile == "decode":
        w = workloads.decode_llama2_7b(dev, num_seqs=16, pool_blocks=4096)
        out = torch.empty_like(w.query)
        for _ in range(3):
            tch_cuda.reshape_and_cache(w.new_key, w.new_value, w.key_cache, w.value_cache, w.slot_mapping)
            tch_cuda.paged_attention_v1(out, w.query, w.key_cache, w.value_cache, w.num_kv_heads, w.scale,
                                        w.block_tables, w.context_lens, 16, w.max_context_len, None)
        torch.cuda.synchronize()
        print(json.dumps({"profile_case": "decode", "seqs": 16, "algorithmic_bytes": w.algorithmic_bytes()}))
    else:
        pw = workloads.prefill_long(dev, seqlen=4096)
        for _ in range(3):
            tch_cuda.flash_attn_varlen(pw.q, pw.k, pw.v, pw.cu_seqlens_q, pw.cu_seqlens_k, pw.max_seqlen_q,
                                       pw.max_seqlen_k, pw.scale, True)
        torch.cuda.synchronize()
        print(json.dumps({"profile_case": "prefill", "seqlen": 4096, "flops": pw.flops()}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="launch the decode step eagerly instead of replaying a CUDA graph")
    ap.add_argument("--gather", default="fused", choices=["fused", "nccl"],
                    help="multi-GPU head-output gather: fused into the attention epilogue (default) or NCCL")
    ap.add_argument("--suite", action="store_true",
                    help="time all five configurations at the current world size and print one JSON object")
    ap.add_argument("--profile", default=None, choices=["decode", "prefill"],
                    help="run a small case three times for a profiler capture and exit")
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
