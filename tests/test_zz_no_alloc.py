"""The allocation-free decode entry point against the ordinary one.

`aici_paged_attention_v1_static` is for callers that cannot allocate device memory when they
call (all spare memory already belongs to the KV pool, or the binding has no allocator): its
scratch is an array inside the library.  The test calls it twice in a row through the C ABI --
the second call on a smaller batch, so stale contents of the shared array from the first call
are still there -- and compares each result with `aici_paged_attention_v1` on the same inputs.
This file sorts last on purpose: a run that stops at the first failure has then already run
every other test.  It passes on its own in a fresh process and after the other tests.
"""
import ctypes

import pytest
import torch

from aici_b200 import _lib, tch_cuda
import workloads

pytestmark = pytest.mark.gpu
MAX_ABS, MEAN_ABS = 2e-2, 2e-3


def _both(dev, w):
    ref = torch.empty_like(w.query)
    tch_cuda.paged_attention_v1(ref, w.query, w.key_cache, w.value_cache, w.num_kv_heads, w.scale,
                                w.block_tables, w.context_lens, 16, w.max_context_len, None)
    got = torch.full_like(w.query, float("nan"))
    tch_cuda.paged_attention_v1_static(got, w.query, w.key_cache, w.value_cache, w.num_kv_heads, w.scale,
                                       w.block_tables, w.context_lens, 16, w.max_context_len, None)
    torch.cuda.synchronize()
    return got.float().cpu(), ref.float().cpu()


def test_static_scratch_entry_point_matches_twice_in_a_row(cuda_device):
    big = workloads.make_decode("a", cuda_device, num_seqs=24, num_heads=32, num_kv_heads=8,
                                ctx_kind="uniform", ctx_lo=1, ctx_hi=3000, pool_blocks=6000, seed=910)
    small = workloads.make_decode("b", cuda_device, num_seqs=5, num_heads=8, num_kv_heads=8,
                                  ctx_kind="uniform", ctx_lo=200, ctx_hi=700, pool_blocks=400, seed=911)
    for w in (big, small):
        got, ref = _both(cuda_device, w)
        assert not torch.isnan(got).any()
        d = (got - ref).abs()
        assert float(d.max()) <= MAX_ABS and float(d.mean()) <= MEAN_ABS, (float(d.max()), float(d.mean()))
    assert _lib.last_status() == 0


def test_static_scratch_entry_point_refuses_oversized_batches(cuda_device):
    need = _lib.lib().aici_paged_attention_workspace_bytes(ctypes.c_int(2048), ctypes.c_int(32),
                                                           ctypes.c_int(8), ctypes.c_int(8192))
    assert need > (32 << 20)
    w = workloads.make_decode("c", cuda_device, num_seqs=2, num_heads=8, num_kv_heads=8,
                              ctx_kind="uniform", ctx_lo=20, ctx_hi=40, pool_blocks=16, seed=912)
    q = w.query[:1].expand(2048, 8, 128).contiguous().repeat(1, 4, 1)  # 2048 seqs x 32 heads
    bt = w.block_tables[:1].expand(2048, -1).contiguous()
    cl = w.context_lens[:1].expand(2048).contiguous()
    out = torch.empty_like(q)
    with pytest.raises(_lib.AiciError, match="built-in array holds"):
        tch_cuda.paged_attention_v1_static(out, q, w.key_cache, w.value_cache, 8, w.scale, bt, cl, 16,
                                           8192, None)
