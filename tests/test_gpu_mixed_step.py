"""Config 5 as one call sequence, the way rLLM issues it (llm/mod.rs:318-354, tmodel.rs:220-232):
reshape_and_cache of every new token (8 prefill chunks of 512 + 192 decode tokens), varlen causal
prefill of the chunks, paged decode of the single-token sequences, then copy_blocks for the AICI
fork of 32 sequences into 4 children each.  Cache contents are checked bit for bit."""
import pytest
import torch

from aici_b200 import _lib, tch_cuda
import workloads
from oracle import cpu_oracle as O

pytestmark = pytest.mark.gpu
MAX_ABS, MEAN_ABS = 2e-2, 2e-3
HQ, HKV, LAYERS = 32, 8, 4


def test_mixed_continuous_batching_step(cuda_device):
    dev = cuda_device
    n_dec, n_chunks, chunk = 192, 8, 512
    ctx = workloads.draw_context_lens("uniform", n_dec, 256, 16384, 5001)
    need = sum((c + 15) // 16 for c in ctx) + n_chunks * (chunk // 16) + 32 * 4 + 8
    pool = need + 64
    # block tables: decode sequences first, then one 32-block run per prefill chunk, rest free
    g = torch.Generator().manual_seed(5002)
    perm = torch.randperm(pool, generator=g).tolist()
    pos, dec_rows = 0, []
    for c in ctx:
        n = (c + 15) // 16
        dec_rows.append(perm[pos:pos + n])
        pos += n
    pre_rows = []
    for _ in range(n_chunks):
        pre_rows.append(perm[pos:pos + chunk // 16])
        pos += chunk // 16
    free = perm[pos:]
    width = max(len(r) for r in dec_rows)
    bt = torch.zeros(n_dec, width, dtype=torch.int32)
    for i, r in enumerate(dec_rows):
        bt[i, :len(r)] = torch.tensor(r, dtype=torch.int32)

    gd = torch.Generator(device=dev).manual_seed(5003)
    kcs = [workloads.randn_bf16((pool, HKV, 16, 16, 8), dev, gd) for _ in range(LAYERS)]
    vcs = [workloads.randn_bf16((pool, HKV, 128, 16), dev, gd) for _ in range(LAYERS)]
    n_tok = n_chunks * chunk + n_dec
    q = workloads.randn_bf16((n_tok, HQ, 128), dev, gd)
    k = workloads.randn_bf16((n_tok, HKV, 128), dev, gd)
    v = workloads.randn_bf16((n_tok, HKV, 128), dev, gd)
    # slot mapping covers all tokens: prefill tokens first (multi-token entries), decode last
    slots = []
    for r in pre_rows:
        slots += [r[t // 16] * 16 + t % 16 for t in range(chunk)]
    slots += [dec_rows[i][(c - 1) // 16] * 16 + (c - 1) % 16 for i, c in enumerate(ctx)]
    slots_t = torch.tensor(slots, dtype=torch.int32, device=dev)
    q_multi = n_chunks * chunk
    scale = 1.0 / 128 ** 0.5

    # ---- layer 0: the whole attention step -----------------------------------------------
    kc, vc = kcs[0], vcs[0]
    kc_ref, vc_ref = kc.cpu(), vc.cpu()
    tch_cuda.reshape_and_cache(k, v, kc, vc, slots_t)
    O.reshape_and_cache(k.cpu(), v.cpu(), kc_ref, vc_ref, slots_t.cpu())
    assert torch.equal(kc.cpu().view(torch.int16), kc_ref.view(torch.int16))
    assert torch.equal(vc.cpu().view(torch.int16), vc_ref.view(torch.int16))

    # prefill chunks: K/V come back out of the cache (gather_cached_kv), GQA handled natively
    gather = torch.tensor(slots[:q_multi], dtype=torch.int32, device=dev)
    kg = torch.empty(q_multi, HKV, 128, dtype=torch.bfloat16, device=dev)
    vg = torch.empty_like(kg)
    tch_cuda.gather_cached_kv(kg, vg, kc, vc, gather)
    assert torch.equal(kg.view(torch.int16), k[:q_multi].view(torch.int16))
    assert torch.equal(vg.view(torch.int16), v[:q_multi].view(torch.int16))
    cu = torch.arange(0, q_multi + 1, chunk, dtype=torch.int32, device=dev)
    y_pre = tch_cuda.flash_attn_varlen(q[:q_multi], kg, vg, cu, cu, chunk, chunk, scale, True)
    want = O.flash_attn_varlen(q[:q_multi].cpu(), kg.cpu(), vg.cpu(), cu.cpu(), cu.cpu(), chunk, chunk, scale, True)
    mx, mean = O.error_stats(y_pre.cpu(), want)
    assert mx <= MAX_ABS and mean <= MEAN_ABS, (mx, mean)

    # the same chunks read straight from the cache through block tables (no gathered copy)
    pre_bt = torch.tensor(pre_rows, dtype=torch.int32, device=dev)
    pre_cl = torch.full((n_chunks,), chunk, dtype=torch.int32, device=dev)
    y_paged = tch_cuda.flash_attn_varlen_paged(q[:q_multi], kc, vc, cu, pre_cl, pre_bt, chunk, chunk, scale, True)
    mx, mean = O.error_stats(y_paged.cpu(), want)
    assert mx <= MAX_ABS and mean <= MEAN_ABS, (mx, mean)
    mx, _ = O.error_stats(y_paged.cpu(), y_pre.float().cpu())
    assert mx <= 1e-2, mx  # two layouts of the same operands: rounding of the last bit at most

    # decode rows: all 192 sequences against the oracle
    y_dec = torch.empty(n_dec, HQ, 128, dtype=torch.bfloat16, device=dev)
    cl = torch.tensor(ctx, dtype=torch.int32, device=dev)
    tch_cuda.paged_attention_v1(y_dec, q[q_multi:], kc, vc, HKV, scale, bt.to(dev), cl, 16, max(ctx), None)
    want = O.paged_attention_v1(q[q_multi:].cpu().contiguous(), kc_ref, vc_ref, HKV, scale, bt, cl.cpu())
    mx, mean = O.error_stats(y_dec.cpu(), want)
    assert mx <= MAX_ABS and mean <= MEAN_ABS, (mx, mean)

    # ---- fork: 32 sequences x 4 children, rLLM copies the shared LAST block per child ------
    mapping = workloads.fork_block_mapping(dec_rows, 32, 4, free)
    assert sum(len(d) for d in mapping.values()) == 128
    before_k = [t.clone() for t in kcs]
    before_v = [t.clone() for t in vcs]
    tch_cuda.copy_blocks(kcs, vcs, mapping)
    torch.cuda.synchronize()
    dsts = sorted(d for ds in mapping.values() for d in ds)
    keep = torch.ones(pool, dtype=torch.bool, device=dev)
    keep[torch.tensor(dsts, device=dev)] = False
    for l in range(LAYERS):
        for s, ds in mapping.items():
            for d in ds:
                assert torch.equal(kcs[l][d].view(torch.int16), before_k[l][s].view(torch.int16))
                assert torch.equal(vcs[l][d].view(torch.int16), before_v[l][s].view(torch.int16))
        # every block that is not a destination is untouched (bitwise, on the device)
        assert torch.equal(kcs[l][keep].view(torch.int16), before_k[l][keep].view(torch.int16))
        assert torch.equal(vcs[l][keep].view(torch.int16), before_v[l][keep].view(torch.int16))
    assert _lib.last_status() == 0
