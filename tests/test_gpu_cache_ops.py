"""GPU parity tests (bit-exact) for reshape_and_cache, gather_cached_kv and copy_blocks,
through the C ABI, against the CPU oracle and the golden fixture."""
import importlib.util
import os

import numpy as np
import pytest
import torch

from aici_b200 import _lib, tch_cuda
import workloads
from oracle import cpu_oracle as O

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def _mg():
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(GOLDEN, "make_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _bits(t):
    return t.detach().cpu().contiguous().view(torch.int16)


def test_golden_fixture(cuda_device):
    mg = _mg()
    c = mg.small_case()
    fx = np.load(os.path.join(GOLDEN, "cache_and_decode_small.npz"))
    d = [str(x) for x in fx["digests"]]
    kc, vc = c["kc"].to(cuda_device), c["vc"].to(cuda_device)
    tch_cuda.reshape_and_cache(c["nk"].to(cuda_device), c["nv"].to(cuda_device), kc, vc,
                               c["slots"].to(cuda_device))
    assert mg.digest(kc.cpu()) == d[0] and mg.digest(vc.cpu()) == d[1]
    out = torch.empty(c["q"].shape, dtype=torch.bfloat16, device=cuda_device)
    tch_cuda.paged_attention_v1(out, c["q"].to(cuda_device), kc, vc, c["hkv"], 1.0 / 128 ** 0.5,
                                c["bt"].to(cuda_device), c["ctx"].to(cuda_device), 16,
                                int(c["ctx"].max()), None)
    mx, mean = O.error_stats(out.cpu(), torch.from_numpy(fx["decode_out"]))
    assert mx <= 2e-2 and mean <= 2e-3, (mx, mean)
    m = fx["block_mapping"].tolist()
    mapping = {}
    for s, t in zip(m[0::2], m[1::2]):
        mapping.setdefault(s, []).append(t)
    tch_cuda.copy_blocks([kc], [vc], mapping)
    assert mg.digest(kc.cpu()) == d[2] and mg.digest(vc.cpu()) == d[3]
    assert _lib.last_status() == 0


@pytest.mark.parametrize("num_tokens,hkv,slot_dtype", [(1, 1, torch.int32), (37, 3, torch.int64),
                                                        (64, 32, torch.int32), (4288, 8, torch.int32)])
def test_reshape_and_gather_bit_exact(cuda_device, num_tokens, hkv, slot_dtype):
    g = torch.Generator().manual_seed(100 + num_tokens)
    nblk = 600 if num_tokens >= 512 else max(8, (num_tokens + 15) // 16 + 5)
    kc = torch.randn(nblk, hkv, 16, 16, 8, generator=g).to(torch.bfloat16)
    vc = torch.randn(nblk, hkv, 128, 16, generator=g).to(torch.bfloat16)
    key = torch.randn(num_tokens, hkv, 128, generator=g).to(torch.bfloat16)
    val = torch.randn(num_tokens, hkv, 128, generator=g).to(torch.bfloat16)
    if num_tokens >= 512:
        # prefill-like: runs of consecutive slots starting at odd offsets, plus scattered decode slots
        blocks = torch.randperm(nblk, generator=g).tolist()
        slots, bi = [], 0
        while len(slots) < num_tokens - 192:
            run = min(512, num_tokens - 192 - len(slots))
            start = 5
            for i in range(run):
                slots.append(blocks[bi + (start + i) // 16] * 16 + (start + i) % 16)
            bi += (start + run + 15) // 16
        rest = [b * 16 + (b % 16) for b in blocks[bi:bi + num_tokens - len(slots)]]
        slots = torch.tensor(slots + rest, dtype=slot_dtype)
    else:
        slots = torch.randperm(nblk * 16, generator=g)[:num_tokens].to(slot_dtype)
    if num_tokens == 37:
        slots[5] = -1  # padding token, skipped
    kc_ref, vc_ref = kc.clone(), vc.clone()
    O.reshape_and_cache(key, val, kc_ref, vc_ref, slots)
    kc_d, vc_d = kc.to(cuda_device), vc.to(cuda_device)
    tch_cuda.reshape_and_cache(key.to(cuda_device), val.to(cuda_device), kc_d, vc_d, slots.to(cuda_device))
    assert torch.equal(_bits(kc_d), _bits(kc_ref))
    assert torch.equal(_bits(vc_d), _bits(vc_ref))
    # inverse
    gs = slots.clamp(min=0).to(torch.int32)
    k_ref, v_ref = torch.zeros_like(key), torch.zeros_like(val)
    O.gather_cached_kv(k_ref, v_ref, kc_ref, vc_ref, gs)
    k_d = torch.zeros_like(key, device=cuda_device)
    v_d = torch.zeros_like(val, device=cuda_device)
    tch_cuda.gather_cached_kv(k_d, v_d, kc_d, vc_d, gs.to(cuda_device))
    assert torch.equal(_bits(k_d), _bits(k_ref)) and torch.equal(_bits(v_d), _bits(v_ref))
    assert _lib.last_status() == 0


def test_reshape_and_cache_strided_tokens(cuda_device):
    g = torch.Generator().manual_seed(5)
    hkv, d = 2, 128
    qkv = torch.randn(19, (4 + 2 + 2) * d, generator=g).to(torch.bfloat16).to(cuda_device)
    key = qkv[:, 4 * d:6 * d].view(19, hkv, d)
    val = qkv[:, 6 * d:8 * d].view(19, hkv, d)
    kc = torch.zeros(6, hkv, 16, 16, 8, dtype=torch.bfloat16, device=cuda_device)
    vc = torch.zeros(6, hkv, 128, 16, dtype=torch.bfloat16, device=cuda_device)
    slots = torch.randperm(96, generator=g)[:19].to(torch.int32)
    tch_cuda.reshape_and_cache(key, val, kc, vc, slots.to(cuda_device))
    kc_ref, vc_ref = torch.zeros_like(kc, device="cpu"), torch.zeros_like(vc, device="cpu")
    O.reshape_and_cache(key.cpu(), val.cpu(), kc_ref, vc_ref, slots)
    assert torch.equal(_bits(kc), _bits(kc_ref)) and torch.equal(_bits(vc), _bits(vc_ref))


def test_bad_slot_is_recorded_not_trapped(cuda_device):
    kc = torch.zeros(2, 1, 16, 16, 8, dtype=torch.bfloat16, device=cuda_device)
    vc = torch.zeros(2, 1, 128, 16, dtype=torch.bfloat16, device=cuda_device)
    key = torch.ones(2, 1, 128, dtype=torch.bfloat16, device=cuda_device)
    slots = torch.tensor([3, 32], dtype=torch.int32, device=cuda_device)  # 32 is one past the end
    tch_cuda.reshape_and_cache(key, key, kc, vc, slots)
    assert _lib.last_status() & 2
    assert _lib.last_status() == 0  # reading clears it
    assert float(kc.float().sum()) == 128.0


@pytest.mark.parametrize("layers,hkv,pairs", [(1, 1, 1), (4, 8, 128), (3, 2, 300)])
def test_copy_blocks_bit_exact_and_isolated(cuda_device, layers, hkv, pairs):
    g = torch.Generator().manual_seed(200 + pairs)
    nblk = 2 * pairs + 8
    kcs = [torch.randn(nblk, hkv, 16, 16, 8, generator=g).to(torch.bfloat16) for _ in range(layers)]
    vcs = [torch.randn(nblk, hkv, 128, 16, generator=g).to(torch.bfloat16) for _ in range(layers)]
    perm = torch.randperm(nblk, generator=g).tolist()
    n_src = max(1, pairs // 4)
    srcs, dsts = perm[:n_src], perm[n_src:n_src + pairs]
    mapping = {}
    for i, dst in enumerate(dsts):
        mapping.setdefault(srcs[i % n_src], []).append(dst)
    kd = [t.to(cuda_device) for t in kcs]
    vd = [t.to(cuda_device) for t in vcs]
    tch_cuda.copy_blocks(kd, vd, mapping)
    O.copy_blocks(kcs, vcs, mapping)
    for l in range(layers):
        assert torch.equal(_bits(kd[l]), _bits(kcs[l])) and torch.equal(_bits(vd[l]), _bits(vcs[l]))
    # the extern's own convention: tables in device memory
    kd2 = [t.clone() for t in kd]
    vd2 = [t.clone() for t in vd]
    flat = []
    for s, ds in {perm[-1]: [perm[-2]]}.items():
        for t in ds:
            flat += [s, t]
    kp = torch.tensor([t.data_ptr() for t in kd2], dtype=torch.int64, device=cuda_device)
    vp = torch.tensor([t.data_ptr() for t in vd2], dtype=torch.int64, device=cuda_device)
    tch_cuda.copy_blocks_2(kp, vp, torch.tensor(flat, dtype=torch.int64, device=cuda_device), kd2[0])
    O.copy_blocks(kcs, vcs, flat)
    for l in range(layers):
        assert torch.equal(_bits(kd2[l]), _bits(kcs[l])) and torch.equal(_bits(vd2[l]), _bits(vcs[l]))
    assert _lib.last_status() == 0


def test_copy_blocks_rejects_out_of_range_pair(cuda_device):
    kc = torch.zeros(4, 1, 16, 16, 8, dtype=torch.bfloat16, device=cuda_device)
    vc = torch.zeros(4, 1, 128, 16, dtype=torch.bfloat16, device=cuda_device)
    with pytest.raises(_lib.AiciError, match="outside the cache"):
        tch_cuda.copy_blocks([kc], [vc], {1: [4]})
