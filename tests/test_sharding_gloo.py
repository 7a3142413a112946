"""World-size-2 CPU tests (gloo) of the KV-head sharding and the head-output gather: each rank
computes its own heads (with the CPU oracle standing in for the kernels) and the gathered result
must equal the unsharded one.  Also the host-side failure paths: bad divisibility, and a rank
that never joins the collective (short process-group timeout) -- for the gather itself and for the
exchange of peer-memory handles that sets up the fused gather."""
import datetime
import os
import socket
import traceback

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from aici_b200 import sharding
import workloads
from oracle import cpu_oracle as O


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _init(rank, world, port, timeout_s=60):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=timeout_s))


def _worker_decode_and_prefill(rank, world, port, q):
    try:
        _init(rank, world, port)
        shard = sharding.current_shard(8, 4)
        assert (shard.rank, shard.world) == (rank, world)
        full = workloads.make_decode("t", "cpu", num_seqs=6, num_heads=8, num_kv_heads=4, ctx_kind="uniform",
                                     ctx_lo=1, ctx_hi=300, pool_blocks=160, seed=50)
        mine = workloads.make_decode("t", "cpu", num_seqs=6, num_heads=8, num_kv_heads=4, ctx_kind="uniform",
                                     ctx_lo=1, ctx_hi=300, pool_blocks=160, seed=50, shard=shard)
        assert torch.equal(mine.block_tables, full.block_tables)
        assert torch.equal(mine.key_cache, sharding.shard_heads(full.key_cache, shard, 1))
        # cache write on the shard, then decode on the shard
        O.reshape_and_cache(mine.new_key, mine.new_value, mine.key_cache, mine.value_cache, mine.slot_mapping)
        O.reshape_and_cache(full.new_key, full.new_value, full.key_cache, full.value_cache, full.slot_mapping)
        assert torch.equal(mine.key_cache, sharding.shard_heads(full.key_cache, shard, 1))
        local = O.paged_attention_v1(mine.query, mine.key_cache, mine.value_cache, mine.num_kv_heads,
                                     mine.scale, mine.block_tables, mine.context_lens)
        want = O.paged_attention_v1(full.query, full.key_cache, full.value_cache, full.num_kv_heads,
                                    full.scale, full.block_tables, full.context_lens)
        got = sharding.gather_heads(local)
        assert got.shape == want.shape and torch.equal(got, want)
        raw = sharding.gather_heads(local, interleave=False)
        assert raw.shape == (world, 6, 4, 128) and torch.equal(raw[rank], local)
        # prefill, GQA group 2
        pf = workloads.make_prefill("p", "cpu", lens_q=[9, 40], lens_k=[30, 40], num_heads=8, num_kv_heads=4,
                                    seed=51)
        pm = workloads.make_prefill("p", "cpu", lens_q=[9, 40], lens_k=[30, 40], num_heads=8, num_kv_heads=4,
                                    seed=51, shard=shard)
        lo = O.flash_attn_varlen(pm.q, pm.k, pm.v, pm.cu_seqlens_q, pm.cu_seqlens_k, 40, 40, pm.scale, True)
        wa = O.flash_attn_varlen(pf.q, pf.k, pf.v, pf.cu_seqlens_q, pf.cu_seqlens_k, 40, 40, pf.scale, True)
        assert torch.equal(sharding.gather_heads(lo), wa)
        dist.barrier()
        dist.destroy_process_group()
        q.put((rank, "ok"))
    except Exception:
        q.put((rank, traceback.format_exc()))


def _worker_missing_rank(rank, world, port, q):
    try:
        _init(rank, world, port, timeout_s=5)
        if rank == 1:
            # this rank fails on the host between steps and never joins the gather
            q.put((rank, "left"))
            q.close()
            q.join_thread()
            os._exit(0)
        x = torch.zeros(4, 2, 128)
        try:
            sharding.gather_heads(x)
            q.put((rank, "gather returned although a rank was missing"))
        except Exception as e:  # the short timeout (or the closed connection) ends the collective
            q.put((rank, "error:" + type(e).__name__))
    except Exception:
        q.put((rank, traceback.format_exc()))
    finally:
        q.close()
        q.join_thread()
        os._exit(0)


def _worker_handle_exchange(rank, world, port, q):
    try:
        _init(rank, world, port)
        got = sharding.exchange_bytes(bytes([rank + 1]) * 64)
        assert got == [bytes([1]) * 64, bytes([2]) * 64], got
        dist.barrier()
        dist.destroy_process_group()
        q.put((rank, "ok"))
    except Exception:
        q.put((rank, traceback.format_exc()))


def _worker_handle_exchange_missing_rank(rank, world, port, q):
    try:
        _init(rank, world, port, timeout_s=5)
        if rank == 1:
            # dies on the host before it published its handle
            q.put((rank, "left"))
            q.close()
            q.join_thread()
            os._exit(0)
        try:
            sharding.exchange_bytes(b"\x07" * 64)
            q.put((rank, "exchange returned although a rank was missing"))
        except sharding.ShardingError as e:
            q.put((rank, "error:" + str(e)[:60]))
    except Exception:
        q.put((rank, traceback.format_exc()))
    finally:
        q.close()
        q.join_thread()
        os._exit(0)


def _run(worker, world=2):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = {}
    for _ in range(world):
        r, msg = q.get(timeout=180)
        results[r] = msg
    for p in procs:
        p.join(timeout=60)
    return results


@pytest.mark.timeout(300)
def test_sharded_path_equals_unsharded_world2():
    res = _run(_worker_decode_and_prefill)
    assert res == {0: "ok", 1: "ok"}, res


@pytest.mark.timeout(300)
def test_missing_rank_is_an_error_not_a_hang():
    res = _run(_worker_missing_rank)
    assert res[1] == "left"
    assert res[0].startswith("error:"), res


@pytest.mark.timeout(300)
def test_handle_exchange_world2():
    res = _run(_worker_handle_exchange)
    assert res == {0: "ok", 1: "ok"}, res


@pytest.mark.timeout(300)
def test_handle_exchange_with_a_missing_rank_is_an_error_string_not_a_hang():
    res = _run(_worker_handle_exchange_missing_rank)
    assert res[1] == "left"
    assert res[0].startswith("error:handle exchange failed"), res


def test_check_world_rejects_bad_divisibility():
    sharding.check_world(32, 8, 8)
    with pytest.raises(sharding.ShardingError, match="divisible"):
        sharding.check_world(32, 8, 3)
    with pytest.raises(sharding.ShardingError):
        sharding.shard_heads(torch.zeros(2, 8, 4), sharding.Shard(0, 3))
    with pytest.raises(sharding.ShardingError, match="initialised process group"):
        sharding.exchange_bytes(b"x")
    assert sharding.current_shard(8, 4).world == 1
    x = torch.randn(3, 4, 8)
    assert torch.equal(sharding.gather_heads(x), x)
