"""GPU parity tests for decode attention over the paged cache (v1 and v2 entry points), through
the C ABI, against the CPU oracle's fp32-softmax result.  Tolerance (stated by the benchmark
definition): max-abs <= 2e-2 and mean-abs <= 2e-3 for bf16 outputs."""
import pytest
import torch

from aici_b200 import _lib, tch_cuda
import workloads
from oracle import cpu_oracle as O

pytestmark = pytest.mark.gpu
MAX_ABS, MEAN_ABS = 2e-2, 2e-3


def _case(seed, hq, hkv, ctx_list, nblk):
    g = torch.Generator().manual_seed(seed)
    kc = torch.randn(nblk, hkv, 16, 16, 8, generator=g).to(torch.bfloat16)
    vc = torch.randn(nblk, hkv, 128, 16, generator=g).to(torch.bfloat16)
    q = torch.randn(len(ctx_list), hq, 128, generator=g).to(torch.bfloat16)
    table, _rows = workloads.build_block_tables(ctx_list, nblk, seed + 1)
    return q, kc, vc, table, torch.tensor(ctx_list, dtype=torch.int32)


def _run_v1(dev, q, kc, vc, hkv, scale, bt, cl):
    out = torch.full(q.shape, float("nan"), dtype=torch.bfloat16, device=dev)
    tch_cuda.paged_attention_v1(out, q.to(dev), kc.to(dev), vc.to(dev), hkv, scale, bt.to(dev),
                                cl.to(dev), 16, int(cl.max()), None)
    return out.cpu()


def _check(got, want):
    assert not torch.isnan(got.float()).any()
    mx, mean = O.error_stats(got, want)
    assert mx <= MAX_ABS and mean <= MEAN_ABS, (mx, mean)


@pytest.mark.parametrize("hq,hkv", [(4, 4), (8, 2), (8, 1), (4, 2)])
def test_edge_context_lengths(cuda_device, hq, hkv):
    ctx = [1, 15, 16, 17, 255, 256, 257, 511, 512, 513, 1000, 0, 3]
    q, kc, vc, bt, cl = _case(300 + hq * 10 + hkv, hq, hkv, ctx, 400)
    scale = 1.0 / 128 ** 0.5
    want = O.paged_attention_v1(q, kc, vc, hkv, scale, bt, cl)
    got = _run_v1(cuda_device, q, kc, vc, hkv, scale, bt, cl)
    _check(got, want)
    assert float(got[ctx.index(0)].float().abs().max()) == 0.0
    assert _lib.last_status() == 0


def test_tail_block_garbage_is_ignored(cuda_device):
    """Cache slots past context_len may hold NaN/Inf (attention_kernels.cu:317-326)."""
    ctx = [5, 33, 250]
    q, kc, vc, bt, cl = _case(311, 8, 2, ctx, 64)
    for i, c in enumerate(ctx):
        blk, off = int(bt[i, (c - 1) // 16]), (c - 1) % 16
        kc[blk, :, :, off + 1:, :] = float("nan")
        vc[blk, :, :, off + 1:] = float("inf")
    scale = 0.09
    want = O.paged_attention_v1(q, kc, vc, 2, scale, bt, cl)
    _check(_run_v1(cuda_device, q, kc, vc, 2, scale, bt, cl), want)


def test_strided_query_rows(cuda_device):
    ctx = [40, 300]
    q, kc, vc, bt, cl = _case(312, 8, 2, ctx, 64)
    fused = torch.zeros(2, 3 * 8 * 128, dtype=torch.bfloat16)
    fused[:, :8 * 128] = q.view(2, -1)
    qd = fused.to(cuda_device)[:, :8 * 128].view(2, 8, 128)
    out = torch.empty(2, 8, 128, dtype=torch.bfloat16, device=cuda_device)
    tch_cuda.paged_attention_v1(out, qd, kc.to(cuda_device), vc.to(cuda_device), 2, 0.1,
                                bt.to(cuda_device), cl.to(cuda_device), 16, 300, None)
    _check(out.cpu(), O.paged_attention_v1(q, kc, vc, 2, 0.1, bt, cl))


def test_large_batch_uses_the_plan_kernel(cuda_device):
    """More than 2048 sequences: the chunk list is built by a separate kernel into the workspace."""
    g = torch.Generator().manual_seed(350)
    ctx = torch.randint(1, 300, (2100,), generator=g).tolist()
    ctx[7] = 0
    q, kc, vc, bt, cl = _case(351, 8, 2, ctx, sum((c + 15) // 16 for c in ctx) + 4)
    got = _run_v1(cuda_device, q, kc, vc, 2, 0.088, bt, cl)
    _check(got, O.paged_attention_v1(q, kc, vc, 2, 0.088, bt, cl))
    assert float(got[7].float().abs().max()) == 0.0
    assert _lib.last_status() == 0


@pytest.mark.parametrize("hq,hkv,ctx", [
    (8, 1, [8000]),                       # one row cut into many pieces: eight warps merge it
    (4, 4, [3000, 0, 0, 1]),              # empty contexts between rows
    (8, 8, [16] * 40 + [5000] + [1] * 30),  # many one-tile rows around a long one
    (32, 8, [37] * 300),                  # more rows than warps: most spans hold several rows
    (8, 2, [0, 0, 0]),                    # nothing to read at all
    (4, 4, [1100 + 13 * i for i in range(64)]),   # 256 rows of about five pieces: four warps merge a row
    (4, 1, [600 + 7 * i for i in range(100)]),    # 400 rows of a few pieces: two warps merge a row
])
def test_span_traversal_shapes(cuda_device, hq, hkv, ctx):
    """The default traversal gives each warp one span of consecutive tiles of the whole batch;
    these batches put the span borders in every position relative to the row borders."""
    nblk = sum((c + 15) // 16 for c in ctx) + 4
    q, kc, vc, bt, cl = _case(360 + len(ctx), hq, hkv, ctx, nblk)
    want = O.paged_attention_v1(q, kc, vc, hkv, 0.088, bt, cl)
    out = torch.full(q.shape, float("nan"), dtype=torch.bfloat16, device=cuda_device)
    tch_cuda.paged_attention_v1(out, q.to(cuda_device), kc.to(cuda_device), vc.to(cuda_device), hkv,
                                0.088, bt.to(cuda_device), cl.to(cuda_device), 16, max(max(ctx), 1), None)
    got = out.cpu()
    _check(got, want)
    for i, c in enumerate(ctx):
        if c == 0:
            assert float(got[i].float().abs().max()) == 0.0
    assert _lib.last_status() == 0


def test_span_and_chunk_traversals_agree(cuda_device):
    """Same batch through both traversals (the chunked one through its own entry point)."""
    w = workloads.make_decode("t", cuda_device, num_seqs=48, num_heads=32, num_kv_heads=8,
                              ctx_kind="loguniform", ctx_lo=16, ctx_hi=4000, pool_blocks=8192, seed=365)
    a, b = torch.empty_like(w.query), torch.empty_like(w.query)
    tch_cuda.paged_attention_v1(a, w.query, w.key_cache, w.value_cache, w.num_kv_heads, w.scale,
                                w.block_tables, w.context_lens, 16, w.max_context_len, None)
    need = _lib.lib().aici_paged_attention_workspace_bytes(48, 32, 8, w.max_context_len)
    tch_cuda.paged_attention_v1_chunked(b, w.query, w.key_cache, w.value_cache, w.num_kv_heads, w.scale,
                                        w.block_tables, w.context_lens, 16, w.max_context_len, 256)
    # the other traversal changed nothing process-wide: the default call still wants the same scratch
    assert _lib.lib().aici_paged_attention_workspace_bytes(48, 32, 8, w.max_context_len) == need
    d = (a.float() - b.float()).abs()
    assert float(d.max()) <= 4e-3, float(d.max())  # same tiles, different split points
    assert _lib.last_status() == 0


@pytest.mark.parametrize("chunk", [0, 16, 64, 512])
def test_chunk_sizes(cuda_device, chunk):
    ctx = [700, 16, 1, 2049, 130]
    q, kc, vc, bt, cl = _case(320, 8, 2, ctx, 300)
    dev = cuda_device
    out = torch.full(q.shape, float("nan"), dtype=torch.bfloat16, device=dev)
    tch_cuda.paged_attention_v1_chunked(out, q.to(dev), kc.to(dev), vc.to(dev), 2, 0.088, bt.to(dev),
                                        cl.to(dev), 16, int(cl.max()), chunk)
    _check(out.cpu(), O.paged_attention_v1(q, kc, vc, 2, 0.088, bt, cl))
    with pytest.raises(_lib.AiciError, match="multiple of 16"):
        tch_cuda.paged_attention_v1_chunked(out, q.to(dev), kc.to(dev), vc.to(dev), 2, 0.088, bt.to(dev),
                                            cl.to(dev), 16, int(cl.max()), 24)


def test_v2_entry_point_and_its_temporaries(cuda_device):
    ctx = [5, 512, 513, 1500, 2048]
    hq, hkv = 8, 2
    q, kc, vc, bt, cl = _case(330, hq, hkv, ctx, 400)
    scale = 1.0 / 128 ** 0.5
    parts = (max(ctx) + 511) // 512
    dev = cuda_device
    out = torch.empty(len(ctx), hq, 128, dtype=torch.bfloat16, device=dev)
    exp_sums = torch.zeros(len(ctx), hq, parts, dtype=torch.float32, device=dev)
    max_logits = torch.zeros(len(ctx), hq, parts, dtype=torch.float32, device=dev)
    tmp_out = torch.zeros(len(ctx), hq, parts, 128, dtype=torch.bfloat16, device=dev)
    tch_cuda.paged_attention_v2(out, exp_sums, max_logits, tmp_out, q.to(dev), kc.to(dev), vc.to(dev),
                                hkv, scale, bt.to(dev), cl.to(dev), 16, max(ctx), None)
    want = O.paged_attention_v2(q, kc, vc, hkv, scale, bt, cl, partition_size=512)
    _check(out.cpu(), want)
    # partition statistics carry the reference's meaning: recombining them on the host gives out
    es, ml, to = exp_sums.cpu(), max_logits.cpu(), tmp_out.cpu().float()
    for s, c in enumerate(ctx):
        n = (c + 511) // 512
        m = ml[s, :, :n].max(dim=1, keepdim=True).values
        w = es[s, :, :n] * torch.exp(ml[s, :, :n] - m)
        rec = (to[s, :, :n] * (w / (w.sum(1, keepdim=True) + 1e-6)).unsqueeze(-1)).sum(1)
        mx, mean = O.error_stats(rec, want[s])
        assert mx <= MAX_ABS and mean <= MEAN_ABS
    assert _lib.last_status() == 0


def test_bad_block_table_entry_is_recorded_not_trapped(cuda_device):
    ctx = [20]
    q, kc, vc, bt, cl = _case(340, 4, 4, ctx, 8)
    bt[0, 1] = 8  # one past the pool
    _run_v1(cuda_device, q, kc, vc, 4, 0.1, bt, cl)
    assert _lib.last_status() & 1
    assert _lib.last_status() == 0


def test_rejects_unsupported_shapes(cuda_device):
    dev = cuda_device
    q = torch.zeros(1, 12, 128, dtype=torch.bfloat16, device=dev)
    kc = torch.zeros(2, 4, 16, 16, 8, dtype=torch.bfloat16, device=dev)
    vc = torch.zeros(2, 4, 128, 16, dtype=torch.bfloat16, device=dev)
    bt = torch.zeros(1, 1, dtype=torch.int32, device=dev)
    cl = torch.ones(1, dtype=torch.int32, device=dev)
    with pytest.raises(_lib.AiciError, match="must be 1, 2, 4 or 8"):
        tch_cuda.paged_attention_v1(torch.empty_like(q), q, kc, vc, 4, 1.0, bt, cl, 16, 1, None)
    with pytest.raises(_lib.AiciError, match="alibi"):
        tch_cuda.paged_attention_v1(torch.empty_like(q), q, kc, vc, 4, 1.0, bt, cl, 16, 1,
                                    torch.zeros(12, device=dev))


@pytest.mark.parametrize("name", ["llama2_7b", "llama3_8b"])
def test_benchmark_configs_full_size(cuda_device, name):
    """Configs 2 and 3 at full size, checked against the oracle on every row, plus the
    cache write of the new tokens (bit-exact on the touched blocks)."""
    w = workloads.decode_llama2_7b(cuda_device) if name == "llama2_7b" else workloads.decode_llama3_8b(cuda_device)
    tch_cuda.reshape_and_cache(w.new_key, w.new_value, w.key_cache, w.value_cache, w.slot_mapping)
    out = torch.empty_like(w.query)
    tch_cuda.paged_attention_v1(out, w.query, w.key_cache, w.value_cache, w.num_kv_heads, w.scale,
                                w.block_tables, w.context_lens, 16, w.max_context_len, None)
    torch.cuda.synchronize()
    assert _lib.last_status() == 0
    kc, vc = w.key_cache.cpu(), w.value_cache.cpu()
    # the written slots hold the new tokens
    nk, nv, slots = w.new_key.cpu(), w.new_value.cpu(), w.slot_mapping.cpu()
    kg, vg = torch.zeros_like(nk), torch.zeros_like(nv)
    O.gather_cached_kv(kg, vg, kc, vc, slots)
    assert torch.equal(kg.view(torch.int16), nk.view(torch.int16))
    assert torch.equal(vg.view(torch.int16), nv.view(torch.int16))
    want = O.paged_attention_v1(w.query.cpu(), kc, vc, w.num_kv_heads, w.scale, w.block_tables.cpu(),
                                w.context_lens.cpu())
    _check(out.cpu(), want)


@pytest.mark.parametrize("hq,hkv,num_seqs,hi", [(32, 32, 64, 4096), (32, 8, 40, 3000), (8, 1, 3, 20000), (4, 4, 300, 60)])
def test_decode_step_equals_cache_write_then_decode(cuda_device, hq, hkv, num_seqs, hi):
    """aici_decode_step (cache write and decode overlapped in one call) against the two separate
    calls on a copy of the same cache: caches bit-identical, outputs bit-identical; several times in
    a row so that the overlap meets different timings.  The new token's slot is read by the decode."""
    dev = cuda_device
    w = workloads.make_decode("s", dev, num_seqs=num_seqs, num_heads=hq, num_kv_heads=hkv, ctx_kind="uniform",
                              ctx_lo=1, ctx_hi=hi, pool_blocks=num_seqs * ((hi + 15) // 16) + 8, seed=400 + hq)
    kc2, vc2 = w.key_cache.clone(), w.value_cache.clone()
    ref = torch.empty_like(w.query)
    tch_cuda.reshape_and_cache(w.new_key, w.new_value, kc2, vc2, w.slot_mapping)
    tch_cuda.paged_attention_v1(ref, w.query, kc2, vc2, hkv, w.scale, w.block_tables, w.context_lens, 16,
                                w.max_context_len, None)
    for rep in range(4):
        kc1, vc1 = w.key_cache.clone(), w.value_cache.clone()
        got = torch.full_like(w.query, float("nan"))
        tch_cuda.decode_step(got, w.new_key, w.new_value, w.slot_mapping, w.query, kc1, vc1, hkv, w.scale,
                             w.block_tables, w.context_lens, 16, w.max_context_len)
        torch.cuda.synchronize()
        assert torch.equal(kc1.view(torch.int16), kc2.view(torch.int16)), rep
        assert torch.equal(vc1.view(torch.int16), vc2.view(torch.int16)), rep
        assert torch.equal(got.view(torch.int16), ref.view(torch.int16)), rep
    want = O.paged_attention_v1(w.query.cpu(), kc2.cpu(), vc2.cpu(), hkv, w.scale, w.block_tables.cpu(),
                                w.context_lens.cpu())
    _check(got.cpu(), want)
    assert _lib.last_status() == 0


def test_decode_step_refuses_a_slot_that_is_not_the_last_position(cuda_device):
    """The overlap is safe only because the write touches nothing but each sequence's last tile: a slot
    anywhere else is recorded and not written."""
    dev = cuda_device
    w = workloads.make_decode("s", dev, num_seqs=5, num_heads=8, num_kv_heads=2, ctx_kind="uniform",
                              ctx_lo=40, ctx_hi=400, pool_blocks=200, seed=411)
    slots = w.slot_mapping.clone()
    slots[2] = int(w.block_tables[2, 0]) * 16 + 3  # first block of the sequence instead of its last position
    slots[4] = -1                                  # a skipped token stays allowed
    kc, vc = w.key_cache.clone(), w.value_cache.clone()
    out = torch.empty_like(w.query)
    tch_cuda.decode_step(out, w.new_key, w.new_value, slots, w.query, kc, vc, 2, w.scale, w.block_tables,
                         w.context_lens, 16, w.max_context_len)
    torch.cuda.synchronize()
    assert _lib.last_status() == 2  # AICI_STATUS_BAD_SLOT
    kc_want, vc_want = w.key_cache.clone(), w.value_cache.clone()
    keep = torch.tensor([0, 1, 3], device=dev)
    tch_cuda.reshape_and_cache(w.new_key[keep].contiguous(), w.new_value[keep].contiguous(), kc_want, vc_want,
                               w.slot_mapping[keep].contiguous())
    assert torch.equal(kc.view(torch.int16), kc_want.view(torch.int16))
    assert torch.equal(vc.view(torch.int16), vc_want.view(torch.int16))
