"""CPU tests of the oracle itself: it must reproduce the reference's stored known-answer test
and agree with the independent PyTorch-CPU port of refkernels.rs."""
import importlib.util
import json
import os

import numpy as np
import pytest
import torch

from oracle import cpu_oracle as O
from oracle import refkernels_cpu as R

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def _load_make_golden():
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(GOLDEN, "make_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_flash_attn_kat_from_reference():
    """rllm/tch-cuda/tests/flash_attn_tests.rs:35-74, reproduced digit for digit."""
    kat = json.load(open(os.path.join(GOLDEN, "flash_attn_kat.json")))
    q = torch.arange(48, dtype=torch.bfloat16).reshape(3, 2, 8)
    k, v, q = q / 40.0, q / 50.0, q / 30.0
    qq, kk, vv = (t.transpose(0, 1).contiguous() for t in (q, k, v))
    cu = torch.tensor([0, 2], dtype=torch.int32)
    out = O.flash_attn_varlen(qq, kk, vv, cu, cu, 32, 32, 0.5, False, p_bf16=True)
    got = O.round_to_bf16(out).float().transpose(0, 1)
    assert got.shape == (3, 2, 8)
    want = torch.tensor(kat["expected"], dtype=torch.float32)
    # the reference rounds to 4 digits in f32 arithmetic; allow half a unit of the last digit
    assert float((torch.round(got * 1e4) / 1e4 - want).abs().max()) <= 1.01e-4


def test_kat_fp32_softmax_within_bound():
    kat = json.load(open(os.path.join(GOLDEN, "flash_attn_kat.json")))
    q = torch.arange(48, dtype=torch.bfloat16).reshape(3, 2, 8)
    k, v, q = q / 40.0, q / 50.0, q / 30.0
    qq, kk, vv = (t.transpose(0, 1).contiguous() for t in (q, k, v))
    cu = torch.tensor([0, 2], dtype=torch.int32)
    out = O.flash_attn_varlen(qq, kk, vv, cu, cu, 32, 32, 0.5, False).transpose(0, 1)
    want = torch.tensor(kat["expected"], dtype=torch.float32)
    mx, mean = O.error_stats(out, want)
    assert mx <= 2e-2 and mean <= 2e-3


def test_golden_small_case_matches_fixture():
    mg = _load_make_golden()
    c = mg.small_case()
    fx = np.load(os.path.join(GOLDEN, "cache_and_decode_small.npz"))
    kc, vc = c["kc"].clone(), c["vc"].clone()
    O.reshape_and_cache(c["nk"], c["nv"], kc, vc, c["slots"])
    d = [str(x) for x in fx["digests"]]
    assert mg.digest(kc) == d[0] and mg.digest(vc) == d[1]
    out = O.paged_attention_v1(c["q"], kc, vc, c["hkv"], R.default_scale(128), c["bt"], c["ctx"])
    assert float((out - torch.from_numpy(fx["decode_out"])).abs().max()) < 2e-5
    O.copy_blocks([kc], [vc], fx["block_mapping"].tolist())
    assert mg.digest(kc) == d[2] and mg.digest(vc) == d[3]


@pytest.mark.parametrize("slot_dtype", [torch.int32, torch.int64])
def test_cache_ops_round_trip_and_port(slot_dtype):
    g = torch.Generator().manual_seed(7)
    nblk, hkv, d, bs, x = 9, 3, 128, 16, 8
    kc = torch.zeros(nblk, hkv, d // x, bs, x, dtype=torch.bfloat16)
    vc = torch.zeros(nblk, hkv, d, bs, dtype=torch.bfloat16)
    n = 37
    slots = torch.randperm(nblk * bs, generator=g)[:n].to(slot_dtype)
    key = torch.randn(n, hkv, d, generator=g).to(torch.bfloat16)
    val = torch.randn(n, hkv, d, generator=g).to(torch.bfloat16)
    kc2, vc2 = kc.clone(), vc.clone()
    O.reshape_and_cache(key, val, kc, vc, slots)
    R.reshape_and_cache(key, val, kc2, vc2, slots)
    assert torch.equal(kc.view(torch.int16), kc2.view(torch.int16))
    assert torch.equal(vc.view(torch.int16), vc2.view(torch.int16))
    k_out, v_out = torch.zeros_like(key), torch.zeros_like(val)
    O.gather_cached_kv(k_out, v_out, kc, vc, slots.to(torch.int32))
    assert torch.equal(k_out.view(torch.int16), key.view(torch.int16))
    assert torch.equal(v_out.view(torch.int16), val.view(torch.int16))
    k_out2, v_out2 = torch.zeros_like(key), torch.zeros_like(val)
    R.gather_cached_kv(k_out2, v_out2, kc, vc, slots.to(torch.int32))
    assert torch.equal(k_out2.view(torch.int16), key.view(torch.int16))


def test_reshape_and_cache_skips_negative_slots_and_strided_tokens():
    g = torch.Generator().manual_seed(8)
    nblk, hkv, d, bs, x = 4, 2, 128, 16, 8
    kc = torch.zeros(nblk, hkv, d // x, bs, x, dtype=torch.bfloat16)
    vc = torch.zeros(nblk, hkv, d, bs, dtype=torch.bfloat16)
    # key/value are column slices of a fused qkv tensor: token stride > heads*d
    qkv = torch.randn(5, (4 + 2 + 2) * d, generator=g).to(torch.bfloat16)
    key = qkv[:, 4 * d:6 * d].view(5, hkv, d)
    val = qkv[:, 6 * d:8 * d].view(5, hkv, d)
    slots = torch.tensor([3, -1, 17, 63, -1], dtype=torch.int64)
    O.reshape_and_cache(key, val, kc, vc, slots)
    k_out, v_out = torch.zeros(5, hkv, d, dtype=torch.bfloat16), torch.zeros(5, hkv, d, dtype=torch.bfloat16)
    O.gather_cached_kv(k_out, v_out, kc, vc, slots.clamp(min=0).to(torch.int32))
    for t, s in enumerate(slots.tolist()):
        if s >= 0:
            assert torch.equal(k_out[t], key[t]) and torch.equal(v_out[t], val[t])
    assert int((kc != 0).sum()) <= 3 * hkv * d


def test_copy_blocks_only_touches_destinations():
    g = torch.Generator().manual_seed(9)
    layers = 3
    kcs = [torch.randn(8, 2, 16, 16, 8, generator=g).to(torch.bfloat16) for _ in range(layers)]
    vcs = [torch.randn(8, 2, 128, 16, generator=g).to(torch.bfloat16) for _ in range(layers)]
    k0 = [t.clone() for t in kcs]
    v0 = [t.clone() for t in vcs]
    O.copy_blocks(kcs, vcs, {1: [4, 5], 2: [7]})
    for l in range(layers):
        for src, dst in ((1, 4), (1, 5), (2, 7)):
            assert torch.equal(kcs[l][dst], k0[l][src]) and torch.equal(vcs[l][dst], v0[l][src])
        for b in (0, 1, 2, 3, 6):
            assert torch.equal(kcs[l][b], k0[l][b]) and torch.equal(vcs[l][b], v0[l][b])
    O.copy_blocks([], [], {1: [2]})  # empty layer list is a no-op, as in lib.rs:283-285


def _decode_case(seed, num_seqs, hq, hkv, ctx_list, nblk):
    g = torch.Generator().manual_seed(seed)
    kc = torch.randn(nblk, hkv, 16, 16, 8, generator=g).to(torch.bfloat16)
    vc = torch.randn(nblk, hkv, 128, 16, generator=g).to(torch.bfloat16)
    q = torch.randn(num_seqs, hq, 128, generator=g).to(torch.bfloat16)
    perm = torch.randperm(nblk, generator=g).tolist()
    width = max((c + 15) // 16 for c in ctx_list)
    bt = torch.zeros(num_seqs, max(width, 1), dtype=torch.int32)
    pos = 0
    for i, c in enumerate(ctx_list):
        n = (c + 15) // 16
        bt[i, :n] = torch.tensor(perm[pos:pos + n], dtype=torch.int32)
        pos += n
    return q, kc, vc, bt, torch.tensor(ctx_list, dtype=torch.int32)


@pytest.mark.parametrize("hq,hkv", [(4, 4), (8, 2), (8, 1)])
def test_paged_attention_oracle_vs_refkernels_port(hq, hkv):
    ctx = [1, 15, 16, 17, 511, 512, 513, 700]
    q, kc, vc, bt, cl = _decode_case(11, len(ctx), hq, hkv, ctx, 160)
    scale = R.default_scale(128)
    a = O.paged_attention_v1(q, kc, vc, hkv, scale, bt, cl)
    b = R.decode_step_cpu(q.float(), kc.float(), vc.float(), hkv, scale, bt, cl, 16)
    assert float((a - b).abs().max()) < 3e-5
    c = O.paged_attention_v2(q, kc, vc, hkv, scale, bt, cl, partition_size=512)
    assert float((a - c).abs().max()) < 3e-5
    # the reference's 16-bit rounding steps stay inside the acceptance bound
    d = O.paged_attention_v1(q, kc, vc, hkv, scale, bt, cl, ref_rounding=True)
    mx, mean = O.error_stats(d, a)
    assert mx <= 2e-2 and mean <= 2e-3


def test_paged_attention_empty_context_is_zero():
    q, kc, vc, bt, cl = _decode_case(12, 2, 4, 4, [0, 5], 8)
    out = O.paged_attention_v1(q, kc, vc, 4, 0.1, bt, cl)
    assert float(out[0].abs().max()) == 0.0 and float(out[1].abs().max()) > 0.0


@pytest.mark.parametrize("lens_q,lens_k", [([64, 128, 37], [64, 128, 37]), ([5, 1, 40], [70, 33, 40]),
                                           ([40], [8])])
def test_varlen_oracle_vs_refkernels_port(lens_q, lens_k):
    g = torch.Generator().manual_seed(13)
    hq, hkv, d = 4, 2, 128
    q = torch.randn(sum(lens_q), hq, d, generator=g).to(torch.bfloat16)
    k = torch.randn(sum(lens_k), hkv, d, generator=g).to(torch.bfloat16)
    v = torch.randn(sum(lens_k), hkv, d, generator=g).to(torch.bfloat16)
    cq = torch.tensor([0] + lens_q).cumsum(0).to(torch.int32)
    ck = torch.tensor([0] + lens_k).cumsum(0).to(torch.int32)
    scale = R.default_scale(d)
    a = O.flash_attn_varlen(q, k, v, cq, ck, max(lens_q), max(lens_k), scale, True)
    if all(lk >= lq for lq, lk in zip(lens_q, lens_k)):
        b = R.varlen_attn(q.float(), R.repeat_kv(k.float(), 2), R.repeat_kv(v.float(), 2), cq, ck,
                          max(lens_q), max(lens_k), scale, True)
        assert float((a - b).abs().max()) < 3e-5
    else:
        # len_k < len_q: the first len_q - len_k rows see nothing and must be zero
        # (flash_fwd_kernel.h:1056); SDPA would give NaN there, so only the oracle is checked
        assert float(a[:lens_q[0] - lens_k[0]].abs().max()) == 0.0
        assert float(a[lens_q[0] - lens_k[0]:].abs().max()) > 0.0
    rows = torch.tensor([[0, 0, 0], [len(lens_q) - 1, sum(lens_q) - 1, hq - 1]], dtype=torch.int32)
    r = O.flash_attn_varlen_rows(q, k, v, cq, ck, rows, scale, True)
    assert torch.allclose(r[0], a[0, 0]) and torch.allclose(r[1], a[-1, hq - 1])


def test_rotary_oracle_vs_refkernels_port():
    g = torch.Generator().manual_seed(21)
    T, hq, hkv, d = 11, 4, 2, 128
    cs = R.make_cos_sin_cache(300, d)
    pos = torch.randint(0, 300, (T,), generator=g)
    q = torch.randn(T, hq * d, generator=g).to(torch.bfloat16)
    k = torch.randn(T, hkv * d, generator=g).to(torch.bfloat16)
    q1, k1 = q.clone(), k.clone()
    O.rotary_embedding(pos, q1, k1, d, cs)
    q2, k2 = q.float(), k.float()
    R.rotary_embedding(pos, q2, k2, d, cs.float())
    # the kernel rounds both products and the sum to bf16 (inputs are ~N(0,1), |x| < 5): each
    # rounding is at most half an ulp of a value below 8, i.e. 2^-6
    for a, b in ((q1, q2), (k1, k2)):
        diff = (a.float() - b).abs()
        assert float(diff.max()) <= 3 * 2.0 ** -6 and float(diff.mean()) <= 5e-3
    # position 0 is the identity (cos 1, sin 0)
    q3, k3 = q.clone(), k.clone()
    O.rotary_embedding(torch.zeros(T, dtype=torch.int64), q3, k3, d, cs)
    assert torch.equal(q3, q) and torch.equal(k3, k)
