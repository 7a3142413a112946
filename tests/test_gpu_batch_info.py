"""The step-metadata builder with its one-copy upload, feeding the kernels it is made for."""
import pytest
import torch

from aici_b200 import _lib, batch_info, tch_cuda
import workloads
from oracle import batch_info_ref
from oracle import cpu_oracle as O

pytestmark = pytest.mark.gpu
BS = 16


def test_device_sections_match_reference_builder(cuda_device):
    from test_batch_info_cpu import check_against_ref, make_entries
    b = batch_info.BatchInfoBuilder(block_size=BS, max_model_len=4096, device=cuda_device)
    for step in range(4):  # staging buffers alternate and are reused
        entries = make_entries(300 + step, 50)
        for e in entries:
            b.add_entry(*e)
        bi = b.finish(step)
        assert bi.tokens.is_cuda and bi.paged_block_tables.is_cuda
        ref = batch_info_ref.finish(entries, BS, 4096)
        check_against_ref(bi, ref)
        assert bi.gather_mapping.tolist() == ref["gather_mapping"]


def test_built_tables_drive_cache_write_and_decode(cuda_device):
    """A decode step described as BatchEntries gives the same bits as the same step with tensors
    made directly, and matches the oracle."""
    w = workloads.make_decode("t", cuda_device, num_seqs=24, num_heads=32, num_kv_heads=8,
                              ctx_kind="uniform", ctx_lo=5, ctx_hi=700, pool_blocks=2048, seed=77)
    tables = w.block_tables.cpu()
    b = batch_info.BatchInfoBuilder(block_size=BS, max_model_len=8192, device=cuda_device,
                                    gather_mapping=False)
    for i, ctx in enumerate(w.context_list):
        slots = [int(tables[i, t // BS]) * BS + t % BS for t in range(ctx)]
        b.add_entry(i, [(ctx - 1, 1)], slots)
    bi = b.finish()
    assert bi.seqlen_multi == 0 and bi.paged_max_context_len == w.max_context_len
    assert torch.equal(bi.slot_mapping, w.slot_mapping)
    assert torch.equal(bi.paged_context_lens, w.context_lens)

    kc1, vc1 = w.key_cache.clone(), w.value_cache.clone()
    kc2, vc2 = w.key_cache.clone(), w.value_cache.clone()
    tch_cuda.reshape_and_cache(w.new_key, w.new_value, kc1, vc1, w.slot_mapping)
    tch_cuda.reshape_and_cache(w.new_key, w.new_value, kc2, vc2, bi.slot_mapping)
    assert torch.equal(kc1.view(torch.int16), kc2.view(torch.int16))
    assert torch.equal(vc1.view(torch.int16), vc2.view(torch.int16))
    out1, out2 = torch.empty_like(w.query), torch.empty_like(w.query)
    tch_cuda.paged_attention_v1(out1, w.query, kc1, vc1, w.num_kv_heads, w.scale, w.block_tables,
                                w.context_lens, BS, w.max_context_len, None)
    tch_cuda.paged_attention_v1(out2, w.query, kc2, vc2, w.num_kv_heads, w.scale,
                                bi.paged_block_tables, bi.paged_context_lens, bi.paged_block_size,
                                bi.paged_max_context_len, None)
    assert torch.equal(out1.view(torch.int16), out2.view(torch.int16))
    want = O.paged_attention_v1(w.query.cpu(), kc1.cpu(), vc1.cpu(), w.num_kv_heads, w.scale,
                                w.block_tables.cpu(), w.context_lens.cpu())
    mx, mean = O.error_stats(out2.cpu(), want)
    assert mx <= 2e-2 and mean <= 2e-3, (mx, mean)
    assert _lib.last_status() == 0


def test_tables_for_all_drive_paged_prefill(cuda_device):
    """Multi-token entries with TABLES_FOR_ALL: the paged prefill reads the context through the
    built rows and equals gather_cached_kv (through the built gather_mapping) + packed prefill."""
    g = torch.Generator().manual_seed(5)
    hq, hkv, nblk = 8, 2, 256
    kc = torch.randn(nblk, hkv, 16, 16, 8, generator=g).to(torch.bfloat16).to(cuda_device)
    vc = torch.randn(nblk, hkv, 128, 16, generator=g).to(torch.bfloat16).to(cuda_device)
    perm = torch.randperm(nblk, generator=g).tolist()
    b = batch_info.BatchInfoBuilder(block_size=BS, max_model_len=8192, device=cuda_device,
                                    tables_for_all=True)
    lens = [(130, 130), (70, 300), (1, 50), (33, 33), (1, 17)]  # (q_len, k_len)
    for i, (ql, kl) in enumerate(lens):
        blocks = [perm.pop() for _ in range((kl + BS - 1) // BS)]
        slots = [blocks[t // BS] * BS + t % BS for t in range(kl)]
        b.add_entry(i, [(kl - ql + j, 7) for j in range(ql)], slots)
    bi = b.finish()
    assert bi.seqlen_multi == 3 and bi.q_multi == 130 + 70 + 33
    q = torch.randn(bi.q_multi, hq, 128, generator=g).to(torch.bfloat16).to(cuda_device)
    scale = 1.0 / 128 ** 0.5
    got = tch_cuda.flash_attn_varlen_paged(q, kc, vc, bi.seqlens_q, bi.multi_context_lens,
                                           bi.multi_block_tables, bi.max_seqlen_q, bi.max_seqlen_k,
                                           scale, True)
    k = torch.empty(bi.gather_mapping.numel(), hkv, 128, dtype=torch.bfloat16, device=cuda_device)
    v = torch.empty_like(k)
    tch_cuda.gather_cached_kv(k, v, kc, vc, bi.gather_mapping)
    want = tch_cuda.flash_attn_varlen(q, k, v, bi.seqlens_q, bi.seqlens_k, bi.max_seqlen_q,
                                      bi.max_seqlen_k, scale, True)
    d = (got.float() - want.float()).abs()
    assert float(d.max()) <= 4e-3, float(d.max())
    ref = O.flash_attn_varlen(q.cpu(), k.cpu(), v.cpu(), bi.seqlens_q.cpu(), bi.seqlens_k.cpu(),
                              bi.max_seqlen_q, bi.max_seqlen_k, scale, True)
    mx, mean = O.error_stats(got.cpu(), ref)
    assert mx <= 2e-2 and mean <= 2e-3, (mx, mean)
    assert _lib.last_status() == 0
