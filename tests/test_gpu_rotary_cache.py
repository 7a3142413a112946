"""GPU parity for rotary embedding fused with the cache write: bit-exact against the CPU oracle
(which restates the reference kernel's bf16 arithmetic) and, in a test of its own that skips when
the comparator library is absent, against the reference's own rotary_embedding + reshape_and_cache
kernels."""
import ctypes
import os

import pytest
import torch

from aici_b200 import _lib, tch_cuda
import workloads
from oracle import cpu_oracle as O
from oracle import refkernels_cpu as R

pytestmark = pytest.mark.gpu
REF_LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref",
                       "libref_vllm.so")


def _bits(t):
    return t.detach().cpu().contiguous().view(torch.int16)


def _inputs(dev, T, hq, hkv, seed):
    g = torch.Generator().manual_seed(seed)
    d, nblk = 128, (T + 15) // 16 + 9
    cs = R.make_cos_sin_cache(4096, d)
    pos = torch.randint(0, 4096, (T,), generator=g)
    qkv = torch.randn(T, (hq + 2 * hkv) * d, generator=g).to(torch.bfloat16)
    kc = torch.randn(nblk, hkv, 16, 16, 8, generator=g).to(torch.bfloat16)
    vc = torch.randn(nblk, hkv, 128, 16, generator=g).to(torch.bfloat16)
    slots = torch.randperm(nblk * 16, generator=g)[:T].to(torch.int32)
    if T > 64:
        slots[:64] = torch.arange(64, dtype=torch.int32) + 19  # a prefill-like run
        slots[64:] = torch.randperm(nblk * 16 - 96, generator=g)[:T - 64].to(torch.int32) + 96
    if T > 3:
        slots[3] = -1
    return cs, pos, qkv, kc, vc, slots


def _ours(dev, T, hq, hkv, cs, pos, qkv, kc, vc, slots):
    """The fused kernel on column slices of the fused projection (strided rows)."""
    d = 128
    qkv_d = qkv.to(dev)
    q = qkv_d[:, :hq * d]
    k = qkv_d[:, hq * d:(hq + hkv) * d]
    v = qkv_d[:, (hq + hkv) * d:]
    kc_d, vc_d = kc.to(dev), vc.to(dev)
    tch_cuda.rotary_embedding_reshape_and_cache(pos.to(dev), q, k, v, d, cs.to(dev), True, kc_d, vc_d,
                                                slots.to(dev))
    torch.cuda.synchronize()
    return q, k, v, kc_d, vc_d


@pytest.mark.parametrize("T,hq,hkv", [(1, 4, 4), (37, 8, 2), (700, 32, 8)])
def test_fused_rotary_cache_bit_exact(cuda_device, T, hq, hkv):
    dev, d = cuda_device, 128
    cs, pos, qkv, kc, vc, slots = _inputs(dev, T, hq, hkv, 40 + T)
    # oracle: rotate, then scatter
    q_ref = qkv[:, :hq * d].clone()  # clone: a one-row column slice is already contiguous
    k_ref = qkv[:, hq * d:(hq + hkv) * d].clone()
    v_ref = qkv[:, (hq + hkv) * d:].clone()
    O.rotary_embedding(pos, q_ref, k_ref, d, cs)
    kc_ref, vc_ref = kc.clone(), vc.clone()
    O.reshape_and_cache(k_ref.view(T, hkv, d), v_ref.view(T, hkv, d), kc_ref, vc_ref, slots)
    q, k, v, kc_d, vc_d = _ours(dev, T, hq, hkv, cs, pos, qkv, kc, vc, slots)
    assert torch.equal(_bits(q), _bits(q_ref)) and torch.equal(_bits(k), _bits(k_ref))
    assert torch.equal(_bits(v), _bits(v_ref))
    assert torch.equal(_bits(kc_d), _bits(kc_ref)) and torch.equal(_bits(vc_d), _bits(vc_ref))
    assert _lib.last_status() == 0


@pytest.mark.parametrize("T,hq,hkv", [(1, 4, 4), (37, 8, 2), (700, 32, 8)])
def test_fused_rotary_cache_vs_reference_kernels(cuda_device, T, hq, hkv):
    """The same call against the reference's own rotary_embedding and reshape_and_cache kernels run
    back to back on the same inputs.  Skipped (visibly) when the comparator library is absent."""
    if not os.path.exists(REF_LIB):
        pytest.skip("reference comparator not built (python oracle/build_ref.py)")
    dev, d = cuda_device, 128
    cs, pos, qkv, kc, vc, slots = _inputs(dev, T, hq, hkv, 40 + T)
    q, k, v, kc_d, vc_d = _ours(dev, T, hq, hkv, cs, pos, qkv, kc, vc, slots)
    ref = ctypes.CDLL(REF_LIB)
    ref.ref_rotary_embedding.restype = ctypes.c_void_p
    ref.ref_reshape_and_cache.restype = ctypes.c_void_p
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    i64 = lambda x: ctypes.c_int64(int(x))
    q2 = qkv[:, :hq * d].clone().to(dev)
    k2 = qkv[:, hq * d:(hq + hkv) * d].clone().to(dev)
    v2 = qkv[:, (hq + hkv) * d:].clone().to(dev)
    kc2, vc2 = kc.to(dev), vc.to(dev)
    pos_d, cs_d = pos.to(dev), cs.to(dev)
    res = ref.ref_rotary_embedding(p(pos_d), p(q2), p(k2), i64(T), i64(hq), i64(hkv), i64(d), p(cs_d),
                                   i64(4096), i64(d), 1, 0)
    assert not res, ctypes.string_at(res)
    s64 = slots.to(torch.int64).to(dev)
    res = ref.ref_reshape_and_cache(p(k2), p(v2), p(kc2), p(vc2), p(s64), i64(T), i64(hkv), i64(d),
                                    i64(kc.shape[0]), i64(16), 0)
    assert not res, ctypes.string_at(res)
    torch.cuda.synchronize()
    assert torch.equal(_bits(q), _bits(q2)) and torch.equal(_bits(k), _bits(k2))
    assert torch.equal(_bits(kc_d), _bits(kc2)) and torch.equal(_bits(vc_d), _bits(vc2))
    assert _lib.last_status() == 0


def test_fused_rotary_rejects_unsupported(cuda_device):
    dev = cuda_device
    cs, pos, qkv, kc, vc, slots = _inputs(dev, 4, 4, 4, 99)
    q, k, v = (t.to(dev).contiguous() for t in (qkv[:, :512], qkv[:, 512:1024], qkv[:, 1024:]))
    with pytest.raises(_lib.AiciError, match="NeoX"):
        tch_cuda.rotary_embedding_reshape_and_cache(pos.to(dev), q, k, v, 128, cs.to(dev), False, kc.to(dev),
                                                    vc.to(dev), slots.to(dev))
    with pytest.raises(_lib.AiciError, match="rot_dim"):
        tch_cuda.rotary_embedding_reshape_and_cache(pos.to(dev), q, k, v, 128, cs[:, :64].contiguous().to(dev),
                                                    True, kc.to(dev), vc.to(dev), slots.to(dev))
