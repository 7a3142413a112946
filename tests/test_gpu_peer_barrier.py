"""The cross-GPU barrier's failure path, exercised on one GPU without any fault: a barrier whose
peer never arrives (a flag that nothing sets) must give up after its bounded wait, record
AICI_STATUS_PEER_TIMEOUT and leave the context usable; one whose peer has arrived passes at once.
The same for the barrier folded into the decode call's last kernel, and: a reported time-out that
nobody has cleared yet must not change what later launches compute."""
import ctypes
import time

import pytest
import torch

from aici_b200 import _lib, tch_cuda
import workloads
from oracle import cpu_oracle as O

pytestmark = pytest.mark.gpu
PEER_TIMEOUT = 8


def _barrier(flags, rank):
    ptrs = (ctypes.c_void_p * len(flags))(*[f.data_ptr() for f in flags])
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    _lib.check("aici_peer_barrier", _lib.lib().aici_peer_barrier(ptrs, ctypes.c_int(len(flags)),
                                                                 ctypes.c_int(rank), stream))


def test_barrier_passes_when_the_peer_has_arrived(cuda_device):
    mine = torch.zeros(32, dtype=torch.int32, device=cuda_device)
    peer = torch.zeros(32, dtype=torch.int32, device=cuda_device)
    mine[1] = 3  # "rank 1" already published epochs 1..3 into rank 0's array
    for epoch in (1, 2, 3):
        t0 = time.perf_counter()
        _barrier([mine, peer], 0)
        torch.cuda.synchronize()
        assert time.perf_counter() - t0 < 0.5
        assert int(peer[0]) == epoch and int(mine[0]) == epoch and int(mine[8]) == epoch
    assert _lib.last_status() == 0


def test_barrier_gives_up_after_its_bounded_wait(cuda_device):
    mine = torch.zeros(32, dtype=torch.int32, device=cuda_device)
    peer = torch.zeros(32, dtype=torch.int32, device=cuda_device)
    t0 = time.perf_counter()
    _barrier([mine, peer], 0)  # nobody will ever write mine[1]
    torch.cuda.synchronize()
    waited = time.perf_counter() - t0
    assert 0.2 < waited < 10.0, waited
    assert _lib.last_status() == PEER_TIMEOUT
    assert _lib.last_status() == 0  # reading clears the word
    # the kernel returned normally: the context works and a later barrier can succeed
    mine[1] = 100
    _barrier([mine, peer], 0)
    torch.cuda.synchronize()
    assert _lib.last_status() == 0
    assert float(torch.ones(8, device=cuda_device).sum()) == 8.0


def test_a_reported_timeout_does_not_change_later_launches(cuda_device):
    """The status word is sticky until somebody reads it; prefill and decode launched while it still
    holds a late peer's time-out must compute exactly what they always compute."""
    dev = cuda_device
    mine = torch.zeros(32, dtype=torch.int32, device=dev)
    peer = torch.zeros(32, dtype=torch.int32, device=dev)
    _barrier([mine, peer], 0)  # times out; the word is NOT read afterwards
    pw = workloads.make_prefill("p", dev, lens_q=[200, 129], lens_k=[328, 129], num_heads=8, num_kv_heads=2,
                                seed=77)
    o = tch_cuda.flash_attn_varlen(pw.q, pw.k, pw.v, pw.cu_seqlens_q, pw.cu_seqlens_k, pw.max_seqlen_q,
                                   pw.max_seqlen_k, pw.scale, True)
    want = O.flash_attn_varlen(pw.q.cpu(), pw.k.cpu(), pw.v.cpu(), pw.cu_seqlens_q.cpu(), pw.cu_seqlens_k.cpu(),
                               pw.max_seqlen_q, pw.max_seqlen_k, pw.scale, True)
    mx, mean = O.error_stats(o.cpu(), want)
    assert mx <= 2e-2 and mean <= 2e-3, (mx, mean)
    w = workloads.make_decode("d", dev, num_seqs=6, num_heads=8, num_kv_heads=2, ctx_kind="uniform",
                              ctx_lo=1, ctx_hi=900, pool_blocks=400, seed=78)
    out = torch.empty_like(w.query)
    tch_cuda.paged_attention_v1(out, w.query, w.key_cache, w.value_cache, w.num_kv_heads, w.scale,
                                w.block_tables, w.context_lens, 16, w.max_context_len, None)
    want = O.paged_attention_v1(w.query.cpu(), w.key_cache.cpu(), w.value_cache.cpu(), w.num_kv_heads, w.scale,
                                w.block_tables.cpu(), w.context_lens.cpu())
    mx, mean = O.error_stats(out.cpu(), want)
    assert mx <= 2e-2 and mean <= 2e-3, (mx, mean)
    assert _lib.last_status() == PEER_TIMEOUT  # only the barrier's bit, still there
    assert _lib.last_status() == 0


def _decode_with_fused_barrier(dev, w, outs, flags, rank):
    tch_cuda.paged_attention_v1_peers([o.data_ptr() for o in outs], w.num_heads, 0, w.query, w.key_cache,
                                      w.value_cache, w.num_kv_heads, w.scale, w.block_tables, w.context_lens,
                                      16, w.max_context_len, barrier_flags=[f.data_ptr() for f in flags],
                                      rank=rank)


def test_barrier_folded_into_the_decode_call(cuda_device):
    """Two "ranks" whose buffers both live on this GPU: the call stores its rows into both output
    buffers; every CTA of its last kernel reports to both ranks (2^20 per call and rank in all, in
    slot 16 + rank) and one CTA waits for both.  First with the peer's reports already there (passes
    at once, twice in a row), then with a peer that never reports (bounded wait, status bit, rows
    still written, context usable)."""
    dev = cuda_device
    w = workloads.make_decode("d", dev, num_seqs=20, num_heads=8, num_kv_heads=2, ctx_kind="uniform",
                              ctx_lo=1, ctx_hi=2500, pool_blocks=4000, seed=79)
    ref = torch.empty_like(w.query)
    tch_cuda.paged_attention_v1(ref, w.query, w.key_cache, w.value_cache, w.num_kv_heads, w.scale,
                                w.block_tables, w.context_lens, 16, w.max_context_len, None)
    mine = torch.zeros(32, dtype=torch.int32, device=dev)
    peer = torch.zeros(32, dtype=torch.int32, device=dev)
    mine[17] = 2 << 20  # "rank 1" has already reported two calls in full
    for epoch in (1, 2):
        outs = [torch.full_like(w.query, float("nan")) for _ in range(2)]
        t0 = time.perf_counter()
        _decode_with_fused_barrier(dev, w, outs, [mine, peer], 0)
        torch.cuda.synchronize()
        assert time.perf_counter() - t0 < 0.5
        assert int(peer[16]) == epoch << 20 and int(mine[16]) == epoch << 20 and int(mine[10]) == epoch
        for o in outs:
            assert torch.equal(o.view(torch.int16), ref.view(torch.int16))
    assert _lib.last_status() == 0
    outs = [torch.full_like(w.query, float("nan")) for _ in range(2)]
    t0 = time.perf_counter()
    _decode_with_fused_barrier(dev, w, outs, [mine, peer], 0)  # call 3: nobody adds to mine[17]
    torch.cuda.synchronize()
    assert 0.2 < time.perf_counter() - t0 < 10.0
    assert _lib.last_status() == PEER_TIMEOUT
    for o in outs:
        assert torch.equal(o.view(torch.int16), ref.view(torch.int16))
    assert int(mine[10]) == 3 and int(mine[16]) == 3 << 20
    assert float(torch.ones(8, device=dev).sum()) == 8.0


def test_barrier_rejects_bad_arguments(cuda_device):
    mine = torch.zeros(32, dtype=torch.int32, device=cuda_device)
    with pytest.raises(_lib.AiciError, match="world must be 1..8"):
        _barrier([mine] * 9, 0)
    with pytest.raises(_lib.AiciError, match="rank inside it"):
        _barrier([mine, mine], 2)
