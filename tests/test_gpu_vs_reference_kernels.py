"""This repository's kernels against the reference's OWN CUDA kernels on the same device buffers.

oracle/_ref/libref_vllm.so holds rllm/tch-cuda/kernels/vllm/cache_kernels.cu and
attention/attention_kernels.cu compiled unmodified for sm_100a (oracle/build_ref.py).  The cache
operations must agree bit for bit; decode attention within the bf16 bound (max-abs 2e-2,
mean-abs 2e-3); the CPU oracle in its reference-rounding mode is checked against the reference
kernel as well, which pins the oracle's restatement of paged attention.  Skipped when the
comparator library has not been built."""
import ctypes
import os

import pytest
import torch

from aici_b200 import _lib, tch_cuda
import workloads
from oracle import cpu_oracle as O

pytestmark = pytest.mark.gpu
REF_LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref",
                       "libref_vllm.so")
MAX_ABS, MEAN_ABS = 2e-2, 2e-3


@pytest.fixture(scope="module")
def ref():
    if not os.path.exists(REF_LIB):
        pytest.skip("reference comparator not built (python oracle/build_ref.py)")
    lib = ctypes.CDLL(REF_LIB)
    for n in ("ref_reshape_and_cache", "ref_gather_cached_kv", "ref_copy_blocks_2", "ref_paged_attention_v1",
              "ref_paged_attention_v2"):
        getattr(lib, n).restype = ctypes.c_void_p
    return lib


def _ok(res):
    if res:
        raise AssertionError(ctypes.string_at(res).decode())


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def _i64(v):
    return ctypes.c_int64(int(v))


def _bits(t):
    return t.contiguous().view(torch.int16)


def test_cache_ops_bit_exact_vs_reference_kernels(cuda_device, ref):
    dev = cuda_device
    g = torch.Generator(device=dev).manual_seed(700)
    nblk, hkv, T = 300, 8, 1000
    kc = workloads.randn_bf16((nblk, hkv, 16, 16, 8), dev, g)
    vc = workloads.randn_bf16((nblk, hkv, 128, 16), dev, g)
    key = workloads.randn_bf16((T, hkv, 128), dev, g)
    val = workloads.randn_bf16((T, hkv, 128), dev, g)
    gc = torch.Generator().manual_seed(701)
    run = torch.arange(600) + 37                                    # a prefill-like run of slots
    scat = torch.randperm(nblk * 16 - 700, generator=gc)[:400] + 700  # scattered decode slots
    slots = torch.cat([run, scat]).to(torch.int32).to(dev)
    kc_r, vc_r = kc.clone(), vc.clone()
    tch_cuda.reshape_and_cache(key, val, kc, vc, slots)
    _ok(ref.ref_reshape_and_cache(_p(key), _p(val), _p(kc_r), _p(vc_r), _p(slots.to(torch.int64)), _i64(T),
                                  _i64(hkv), _i64(128), _i64(nblk), _i64(16), 0))
    torch.cuda.synchronize()
    assert torch.equal(_bits(kc), _bits(kc_r)) and torch.equal(_bits(vc), _bits(vc_r))

    k1, v1 = torch.zeros_like(key), torch.zeros_like(val)
    k2, v2 = torch.zeros_like(key), torch.zeros_like(val)
    tch_cuda.gather_cached_kv(k1, v1, kc, vc, slots)
    _ok(ref.ref_gather_cached_kv(_p(k2), _p(v2), _p(kc), _p(vc), _p(slots), _i64(T), _i64(hkv), _i64(128),
                                 _i64(nblk), _i64(16), 0))
    torch.cuda.synchronize()
    assert torch.equal(_bits(k1), _bits(k2)) and torch.equal(_bits(v1), _bits(v2))
    assert torch.equal(_bits(k1), _bits(key))

    # copy_blocks: 3 layers, 40 pairs
    layers = 3
    kcs = [workloads.randn_bf16((nblk, hkv, 16, 16, 8), dev, g) for _ in range(layers)]
    vcs = [workloads.randn_bf16((nblk, hkv, 128, 16), dev, g) for _ in range(layers)]
    kcs_r = [t.clone() for t in kcs]
    vcs_r = [t.clone() for t in vcs]
    perm = torch.randperm(nblk, generator=gc).tolist()
    mapping = {perm[i]: [perm[10 + 4 * i + c] for c in range(4)] for i in range(10)}
    tch_cuda.copy_blocks(kcs, vcs, mapping)
    flat = torch.tensor([x for s, ds in mapping.items() for d in ds for x in (s, d)], dtype=torch.int64, device=dev)
    kp = torch.tensor([t.data_ptr() for t in kcs_r], dtype=torch.int64, device=dev)
    vp = torch.tensor([t.data_ptr() for t in vcs_r], dtype=torch.int64, device=dev)
    _ok(ref.ref_copy_blocks_2(_p(kp), _p(vp), _p(flat), _i64(layers), _i64(40), _p(kcs_r[0]), _i64(nblk),
                              _i64(hkv), _i64(128), _i64(16), 0))
    torch.cuda.synchronize()
    for l in range(layers):
        assert torch.equal(_bits(kcs[l]), _bits(kcs_r[l])) and torch.equal(_bits(vcs[l]), _bits(vcs_r[l]))
    assert _lib.last_status() == 0


@pytest.mark.parametrize("hq,hkv,kind,lo,hi", [(32, 32, "uniform", 512, 4096), (32, 8, "loguniform", 128, 8192),
                                                (8, 8, "uniform", 1, 40)])
def test_paged_attention_v1_vs_reference_kernel(cuda_device, ref, hq, hkv, kind, lo, hi):
    dev = cuda_device
    w = workloads.make_decode("r", dev, num_seqs=24, num_heads=hq, num_kv_heads=hkv, ctx_kind=kind,
                              ctx_lo=lo, ctx_hi=hi, pool_blocks=8192, seed=710 + hkv)
    S = w.query.shape[0]
    mine = torch.empty_like(w.query)
    tch_cuda.paged_attention_v1(mine, w.query, w.key_cache, w.value_cache, hkv, w.scale, w.block_tables,
                                w.context_lens, 16, w.max_context_len, None)
    theirs = torch.empty_like(w.query)
    _ok(ref.ref_paged_attention_v1(_p(theirs), _p(w.query), _p(w.key_cache), _p(w.value_cache), hkv,
                                   ctypes.c_float(w.scale), _p(w.block_tables), _p(w.context_lens), 16,
                                   w.max_context_len, _i64(S), _i64(hq), _i64(128),
                                   _i64(w.block_tables.shape[1]), _i64(w.key_cache.shape[0]), 0))
    torch.cuda.synchronize()
    mx, mean = O.error_stats(mine.cpu(), theirs.cpu().float())
    assert mx <= MAX_ABS and mean <= MEAN_ABS, (mx, mean)
    # the oracle's restatement of the reference kernel (with its 16-bit rounding steps)
    orc = O.paged_attention_v1(w.query.cpu(), w.key_cache.cpu(), w.value_cache.cpu(), hkv, w.scale,
                               w.block_tables.cpu(), w.context_lens.cpu(), ref_rounding=True)
    mx2, mean2 = O.error_stats(theirs.cpu(), orc)
    ulp = float(theirs.float().abs().max()) * 2.0 ** -7  # one bf16 ulp at the largest output
    assert mx2 <= max(8e-3, ulp) and mean2 <= 1e-3, (mx2, mean2, ulp)
    # and the fp32-softmax oracle sits between both
    exact = O.paged_attention_v1(w.query.cpu(), w.key_cache.cpu(), w.value_cache.cpu(), hkv, w.scale,
                                 w.block_tables.cpu(), w.context_lens.cpu())
    mx3, mean3 = O.error_stats(theirs.cpu(), exact)
    assert mx3 <= MAX_ABS and mean3 <= MEAN_ABS, (mx3, mean3)


def test_paged_attention_v2_vs_reference_kernel(cuda_device, ref):
    dev = cuda_device
    hq, hkv = 32, 8
    w = workloads.make_decode("r2", dev, num_seqs=16, num_heads=hq, num_kv_heads=hkv, ctx_kind="uniform",
                              ctx_lo=100, ctx_hi=3000, pool_blocks=4096, seed=720)
    S, parts = w.query.shape[0], (w.max_context_len + 511) // 512

    def bufs():
        return (torch.empty_like(w.query), torch.zeros(S, hq, parts, device=dev),
                torch.zeros(S, hq, parts, device=dev),
                torch.zeros(S, hq, parts, 128, dtype=torch.bfloat16, device=dev))
    o1, es1, ml1, to1 = bufs()
    tch_cuda.paged_attention_v2(o1, es1, ml1, to1, w.query, w.key_cache, w.value_cache, hkv, w.scale,
                                w.block_tables, w.context_lens, 16, w.max_context_len, None)
    o2, es2, ml2, to2 = bufs()
    _ok(ref.ref_paged_attention_v2(_p(o2), _p(es2), _p(ml2), _p(to2), _p(w.query), _p(w.key_cache),
                                   _p(w.value_cache), hkv, ctypes.c_float(w.scale), _p(w.block_tables),
                                   _p(w.context_lens), 16, w.max_context_len, _i64(S), _i64(hq), _i64(128),
                                   _i64(w.block_tables.shape[1]), _i64(w.key_cache.shape[0]), 0))
    torch.cuda.synchronize()
    mx, mean = O.error_stats(o1.cpu(), o2.cpu().float())
    assert mx <= MAX_ABS and mean <= MEAN_ABS, (mx, mean)
    # the caller-visible temporaries carry the same meaning for every partition that holds tokens
    for s, c in enumerate(w.context_list):
        n = (c + 511) // 512
        assert torch.allclose(ml1[s, :, :n], ml2[s, :, :n], atol=2e-3, rtol=1e-3)
        assert torch.allclose(es1[s, :, :n], es2[s, :, :n], atol=1e-3, rtol=5e-3)
        mx_t, mean_t = O.error_stats(to1[s, :, :n].cpu(), to2[s, :, :n].cpu().float())
        assert mx_t <= MAX_ABS and mean_t <= MEAN_ABS
