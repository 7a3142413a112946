"""Multi-GPU parity: KV heads sharded over 2/4/8 GPUs of one box (one process per GPU, NCCL),
head outputs gathered, result compared on rank 0 with the CPU oracle on the UNSHARDED problem; the
fused gather (peer buffers mapped through the C ABI alone) must reproduce the NCCL gather bit for
bit over consecutive steps.  Skipped on a single-GPU box.  Every rank draws the same full tensors
and keeps its heads."""
import os
import socket
import traceback

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
MAX_ABS, MEAN_ABS = 2e-2, 2e-3


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    try:
        import torch.distributed as dist
        from aici_b200 import _lib, sharding, tch_cuda
        import workloads
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dev = torch.device("cuda", rank)
        torch.cuda.set_device(dev)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
        report = {}

        def decode_case(name, **kw):
            shard = sharding.current_shard(kw["num_heads"], kw["num_kv_heads"])
            w = workloads.make_decode(name, dev, shard=shard, **kw)
            kc0, vc0 = w.key_cache.clone(), w.value_cache.clone()  # the cache before this step's tokens
            tch_cuda.reshape_and_cache(w.new_key, w.new_value, w.key_cache, w.value_cache, w.slot_mapping)
            # three consecutive steps with different queries: NCCL gather as the comparison ...
            queries = [w.query, (w.query * 2).contiguous(), (w.query * 0.5).contiguous()]
            fulls = []
            for qk in queries:
                out = torch.empty_like(qk)
                tch_cuda.paged_attention_v1(out, qk, w.key_cache, w.value_cache, w.num_kv_heads, w.scale,
                                            w.block_tables, w.context_lens, 16, w.max_context_len, None)
                fulls.append(sharding.gather_heads(out).contiguous())
            # ... and the fused epilogue: rows stored straight into every rank's buffer (mapped through
            # the library's own peer-memory calls), two buffers used in turn, a reader on the stream
            # between the steps, the barrier once as a launch of its own and twice folded into the call
            pg = sharding.PeerGather(w.query.shape[0], kw["num_heads"], 128, dev)
            pg.barrier()
            snaps = []
            for step, qk in enumerate(queries):
                fold = step > 0
                tch_cuda.paged_attention_v1_peers(pg.ptrs, kw["num_heads"], pg.head0, qk, w.key_cache,
                                                  w.value_cache, w.num_kv_heads, w.scale, w.block_tables,
                                                  w.context_lens, 16, w.max_context_len,
                                                  barrier_flags=pg.flag_ptrs if fold else None, rank=pg.rank)
                if not fold:
                    pg.barrier()
                snaps.append(pg.tensor.clone())  # the reader
                pg.flip()
            torch.cuda.synchronize()
            for step, (snap, full) in enumerate(zip(snaps, fulls)):
                assert torch.equal(snap.view(torch.int16), full.view(torch.int16)), "%s fused gather, step %d" % (name, step)
            # the gather as a call of its own
            out = torch.empty_like(w.query)
            tch_cuda.paged_attention_v1(out, w.query, w.key_cache, w.value_cache, w.num_kv_heads, w.scale,
                                        w.block_tables, w.context_lens, 16, w.max_context_len, None)
            tch_cuda.gather_heads(pg.ptrs, kw["num_heads"], pg.head0, out)
            pg.barrier()
            torch.cuda.synchronize()
            assert torch.equal(pg.tensor.view(torch.int16), fulls[0].view(torch.int16)), name + " gather_heads"
            # the whole step as one call: cache write inside the decode kernel, gather, barrier
            pg.flip()
            tch_cuda.decode_step(None, w.new_key, w.new_value, w.slot_mapping, w.query, kc0, vc0, w.num_kv_heads,
                                 w.scale, w.block_tables, w.context_lens, 16, w.max_context_len, peer_ptrs=pg.ptrs,
                                 barrier_flags=pg.flag_ptrs, rank=pg.rank, total_heads=kw["num_heads"],
                                 head0=pg.head0)
            torch.cuda.synchronize()
            assert torch.equal(pg.tensor.view(torch.int16), fulls[0].view(torch.int16)), name + " decode_step"
            assert torch.equal(kc0.view(torch.int16), w.key_cache.view(torch.int16)), name + " decode_step key cache"
            assert torch.equal(vc0.view(torch.int16), w.value_cache.view(torch.int16)), name + " decode_step value cache"
            pg.close()
            full = fulls[0]
            if rank == 0:
                from oracle import cpu_oracle as O
                f = workloads.make_decode(name, dev, **kw)  # unsharded, same seed
                kc, vc = f.key_cache.cpu(), f.value_cache.cpu()
                O.reshape_and_cache(f.new_key.cpu(), f.new_value.cpu(), kc, vc, f.slot_mapping.cpu())
                want = O.paged_attention_v1(f.query.cpu(), kc, vc, f.num_kv_heads, f.scale,
                                            f.block_tables.cpu(), f.context_lens.cpu())
                report[name] = O.error_stats(full.cpu(), want)

        def prefill_case(name, **kw):
            shard = sharding.current_shard(kw["num_heads"], kw["num_kv_heads"])
            w = workloads.make_prefill(name, dev, shard=shard, **kw)
            o = tch_cuda.flash_attn_varlen(w.q, w.k, w.v, w.cu_seqlens_q, w.cu_seqlens_k, w.max_seqlen_q,
                                           w.max_seqlen_k, w.scale, True)
            full = sharding.gather_heads(o)
            pg = sharding.PeerGather(w.q.shape[0], kw["num_heads"], 128, dev)
            pg.barrier()
            for _ in range(2):  # both buffers
                tch_cuda.flash_attn_varlen_peers(pg.ptrs, kw["num_heads"], pg.head0, w.q, w.k, w.v, w.cu_seqlens_q,
                                                 w.cu_seqlens_k, w.max_seqlen_q, w.max_seqlen_k, w.scale, True)
                pg.barrier()
                torch.cuda.synchronize()
                assert torch.equal(pg.tensor.view(torch.int16), full.contiguous().view(torch.int16)), name + " fused gather"
                pg.flip()
            pg.close()
            if rank == 0:
                from oracle import cpu_oracle as O
                f = workloads.make_prefill(name, dev, **kw)
                want = O.flash_attn_varlen(f.q.cpu(), f.k.cpu(), f.v.cpu(), f.cu_seqlens_q.cpu(),
                                           f.cu_seqlens_k.cpu(), f.max_seqlen_q, f.max_seqlen_k, f.scale, True)
                report[name] = O.error_stats(full.cpu(), want)

        # config 2 / 3 / 5-decode shapes at a size the CPU checks in seconds
        decode_case("cfg2_mha32", num_seqs=16, num_heads=32, num_kv_heads=32, ctx_kind="uniform",
                    ctx_lo=512, ctx_hi=4096, pool_blocks=4096, seed=2000)
        decode_case("cfg3_gqa32_8", num_seqs=48, num_heads=32, num_kv_heads=8, ctx_kind="loguniform",
                    ctx_lo=128, ctx_hi=8192, pool_blocks=12288, seed=3000)
        decode_case("cfg5_decode_gqa32_8", num_seqs=12, num_heads=32, num_kv_heads=8, ctx_kind="uniform",
                    ctx_lo=256, ctx_hi=16384, pool_blocks=8192, seed=5000)
        # config 1 full, config 4 shape at 2 x 1024, config 5 chunks with 1024 cached tokens
        prefill_case("cfg1", lens_q=[64, 128, 256, 512], lens_k=[64, 128, 256, 512], num_heads=32,
                     num_kv_heads=32, seed=1000)
        prefill_case("cfg4_gqa64_8", lens_q=[1024, 1024], lens_k=[1024, 1024], num_heads=64, num_kv_heads=8,
                     seed=4000)
        prefill_case("cfg5_chunks_cached", lens_q=[512] * 2, lens_k=[1536] * 2, num_heads=32, num_kv_heads=8,
                     seed=5100)
        torch.cuda.synchronize()
        status = _lib.last_status()
        dist.barrier()
        dist.destroy_process_group()
        q.put((rank, "ok", status, report))
    except Exception:
        q.put((rank, traceback.format_exc(), -1, {}))


@pytest.mark.parametrize("world", [2, 4, 8])
def test_sharded_configs_match_oracle(world):
    if not torch.cuda.is_available() or torch.cuda.device_count() < world:
        pytest.skip("needs %d GPUs" % world)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=900) for _ in range(world)]
    for p in procs:
        p.join(timeout=120)
    for rank, msg, status, _rep in res:
        assert msg == "ok", "rank %d: %s" % (rank, msg)
        assert status == 0
    report = [r for r in res if r[0] == 0][0][3]
    assert len(report) == 6
    print("world", world, {k: ("%.2e" % v[0], "%.2e" % v[1]) for k, v in report.items()})
    for name, (mx, mean) in report.items():
        assert mx <= MAX_ABS and mean <= MEAN_ABS, (name, mx, mean)
