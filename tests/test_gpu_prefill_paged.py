"""GPU parity tests for prefill attention that reads K/V from the paged cache through block
tables (the gather_cached_kv + repeat_kv + flash_attn_varlen sequence of rLLM in one call).
Checked against the CPU oracle (gather on the CPU, then fp32-softmax varlen attention) and
against this repository's packed-K/V kernel.  Tolerance: max-abs 2e-2, mean-abs 2e-3."""
import pytest
import torch

from aici_b200 import _lib, tch_cuda
import workloads
from oracle import cpu_oracle as O

pytestmark = pytest.mark.gpu
MAX_ABS, MEAN_ABS = 2e-2, 2e-3


def _case(dev, seed, lens_q, lens_k, hq, hkv, poison_tail=False):
    g = torch.Generator().manual_seed(seed)
    nblk = sum((k + 15) // 16 for k in lens_k) + 7
    table, rows = workloads.build_block_tables(lens_k, nblk, seed + 1, first_block=1)
    gd = torch.Generator(device=dev).manual_seed(seed + 2)
    kc = workloads.randn_bf16((nblk, hkv, 16, 16, 8), dev, gd)
    vc = workloads.randn_bf16((nblk, hkv, 128, 16), dev, gd)
    q = workloads.randn_bf16((sum(lens_q), hq, 128), dev, gd)
    if poison_tail:
        for r, k in zip(rows, lens_k):
            off = k % 16
            if off:
                kc[r[-1], :, :, off:, :] = float("nan")
                vc[r[-1], :, :, off:] = float("nan")
        kc[0] = float("nan")  # block 0 is never referenced
        vc[0] = float("inf")
    cu_q = torch.tensor([0] + lens_q).cumsum(0).to(torch.int32)
    cl = torch.tensor(lens_k, dtype=torch.int32)
    slots = torch.tensor([r[t // 16] * 16 + t % 16 for r, k in zip(rows, lens_k) for t in range(k)],
                         dtype=torch.int32)
    return q, kc, vc, table, cu_q, cl, slots


def _oracle(q, kc, vc, cu_q, lens_k, slots, scale, hkv):
    kcc, vcc = kc.cpu(), vc.cpu()
    k = torch.zeros(sum(lens_k), hkv, 128, dtype=torch.bfloat16)
    v = torch.zeros_like(k)
    O.gather_cached_kv(k, v, kcc, vcc, slots)
    cu_k = torch.tensor([0] + lens_k).cumsum(0).to(torch.int32)
    lq = (cu_q[1:] - cu_q[:-1]).tolist()
    want = O.flash_attn_varlen(q.cpu(), k, v, cu_q, cu_k, max(lq), max(lens_k), scale, True)
    return want, k, v, cu_k


@pytest.mark.parametrize("lens_q,lens_k,hq,hkv,poison", [
    ([128, 256], [128, 256], 4, 4, False),              # fresh prompts, block-aligned
    ([1, 37, 130, 300], [1, 37, 130, 300], 8, 2, True),  # ragged, partial last blocks hold NaN
    ([512] * 3, [1536] * 3, 8, 2, False),               # config-5 variant: 1024 tokens already cached
    ([5, 64, 200], [77, 1000, 215], 4, 1, True),        # chunked prefill, odd lengths
])
@pytest.mark.parametrize("max_k", [pytest.param(None, id="shape_by_length"), pytest.param(4096, id="two_tile_shape")])
def test_paged_prefill_matches_oracle_and_packed_kernel(cuda_device, lens_q, lens_k, hq, hkv, poison, max_k):
    """max_k: the upper bound on the context length the caller passes; it selects the kernel shape
    (one query tile per CTA up to 1024 keys, two above), so a loose bound runs the other shape."""
    dev = cuda_device
    q, kc, vc, table, cu_q, cl, slots = _case(dev, 900 + hq, lens_q, lens_k, hq, hkv, poison)
    scale = 1.0 / 128 ** 0.5
    out = tch_cuda.flash_attn_varlen_paged(q, kc, vc, cu_q.to(dev), cl.to(dev), table.to(dev), max(lens_q),
                                           max_k or max(lens_k), scale, True)
    torch.cuda.synchronize()
    assert _lib.last_status() == 0
    want, k, v, cu_k = _oracle(q, kc, vc, cu_q, lens_k, slots, scale, hkv)
    got = out.cpu()
    assert torch.isfinite(got.float()).all()
    mx, mean = O.error_stats(got, want)
    assert mx <= MAX_ABS and mean <= MEAN_ABS, (mx, mean)
    packed = tch_cuda.flash_attn_varlen(q, k.to(dev), v.to(dev), cu_q.to(dev), cu_k.to(dev), max(lens_q),
                                        max_k or max(lens_k), scale, True)
    mx2, mean2 = O.error_stats(got, packed.cpu().float())
    assert mx2 <= 4e-3 and mean2 <= 1e-4, (mx2, mean2)  # same arithmetic, different staging


def test_paged_prefill_after_reshape_and_cache(cuda_device):
    """The rLLM order: write the new tokens into the cache, then attend through the block table."""
    dev = cuda_device
    lens = [200, 513]
    q, kc, vc, table, cu_q, cl, slots = _case(dev, 950, lens, lens, 8, 2)
    g = torch.Generator(device=dev).manual_seed(951)
    k = workloads.randn_bf16((sum(lens), 2, 128), dev, g)
    v = workloads.randn_bf16((sum(lens), 2, 128), dev, g)
    tch_cuda.reshape_and_cache(k, v, kc, vc, slots.to(dev))
    out = tch_cuda.flash_attn_varlen_paged(q, kc, vc, cu_q.to(dev), cl.to(dev), table.to(dev), max(lens),
                                           max(lens), 0.09, True)
    want = O.flash_attn_varlen(q.cpu(), k.cpu(), v.cpu(), cu_q, cu_q, max(lens), max(lens), 0.09, True)
    mx, mean = O.error_stats(out.cpu(), want)
    assert mx <= MAX_ABS and mean <= MEAN_ABS, (mx, mean)


def test_paged_prefill_bad_block_is_recorded(cuda_device):
    dev = cuda_device
    q, kc, vc, table, cu_q, cl, slots = _case(dev, 960, [40], [40], 4, 4)
    table[0, 1] = kc.shape[0]  # one past the pool
    tch_cuda.flash_attn_varlen_paged(q, kc, vc, cu_q.to(dev), cl.to(dev), table.to(dev), 40, 40, 0.1, True)
    assert _lib.last_status() & 1
