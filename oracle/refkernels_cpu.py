"""PyTorch-CPU restatement of rLLM's CPU kernels -- TEST INFRASTRUCTURE / CPU BASELINE ONLY.

Op-for-op port of rllm/rllm-cuda/src/llm/refkernels.rs (the path rLLM runs when built
without the ``cuda`` feature) to the Python front-end of the same ATen operators.  The
Rust original cannot be compiled in this image (no cargo), so this port is what the
benchmark times as the CPU baseline (kind "port") and what the tests use as a second,
independent restatement next to the C oracle.
"""
import math

import torch


def reshape_and_cache(key, value, key_cache, value_cache, slot_mapping):
    """refkernels.rs:5-30: one indexed copy_ per token."""
    _nb, num_heads, head_size_x, block_size, x = key_cache.shape
    key_reshaped = key.reshape(-1, num_heads, head_size_x, x)
    for idx, slot in enumerate(slot_mapping.tolist()):
        block_idx, block_off = slot // block_size, slot % block_size
        key_cache[block_idx, :, :, block_off, :].copy_(key_reshaped[idx])
        value_cache[block_idx, :, :, block_off].copy_(value[idx])


def gather_cached_kv(key, value, key_cache, value_cache, slot_mapping):
    """refkernels.rs:32-57."""
    _nb, num_heads, head_size_x, block_size, x = key_cache.shape
    key_reshaped = key.view(-1, num_heads, head_size_x, x)
    for idx, slot in enumerate(slot_mapping.tolist()):
        block_idx, block_off = slot // block_size, slot % block_size
        key_reshaped[idx].copy_(key_cache[block_idx, :, :, block_off, :])
        value[idx].copy_(value_cache[block_idx, :, :, block_off])


def varlen_attn(q, k, v, seqlens_q, seqlens_k, max_seqlen_q, max_seqlen_k, softmax_scale, causal):
    """refkernels.rs:59-148: per sequence, additive bottom-right causal bias, then
    scaled_dot_product_attention.  k and v must already have as many heads as q (rLLM calls
    repeat_kv first, llm/mod.rs:214-215)."""
    seqlens_q = seqlens_q.tolist()
    seqlens_k = seqlens_k.tolist()
    assert len(seqlens_q) == len(seqlens_k)
    assert causal
    num_heads, head_dim = q.shape[1], q.shape[2]
    attns = []
    for i in range(len(seqlens_k) - 1):
        ptr_q, ptr_k = seqlens_q[i], seqlens_k[i]
        len_q, len_k = seqlens_q[i + 1] - ptr_q, seqlens_k[i + 1] - ptr_k
        assert len_q <= max_seqlen_q and len_k <= max_seqlen_k
        qi = q[ptr_q:ptr_q + len_q].transpose(0, 1)
        ki = k[ptr_k:ptr_k + len_k].transpose(0, 1)
        vi = v[ptr_k:ptr_k + len_k].transpose(0, 1)
        attn_bias = torch.zeros(len_q, len_k, dtype=q.dtype)
        mask = torch.ones(len_q, len_q, dtype=torch.bool).tril(0).logical_not()
        attn_bias[:, len_k - len_q:].masked_fill_(mask, float("-inf"))
        a = torch.nn.functional.scaled_dot_product_attention(
            qi, ki, vi, attn_mask=attn_bias, dropout_p=0.0, is_causal=False, scale=softmax_scale)
        attns.append(a.reshape(num_heads, len_q, head_dim).transpose(0, 1))
    return torch.cat(attns, 0)


def repeat_kv(x, n_rep):
    """llm/mod.rs:357-365."""
    return x if n_rep == 1 else x.repeat_interleave(n_rep, dim=1)


def rotary_embedding(positions, query0, key0, head_size, cos_sin_cache, is_neox=True):
    """refkernels.rs:150-211, NeoX only (the other branch is todo!() there).  In place."""
    assert is_neox
    rot_dim = cos_sin_cache.shape[1]
    num_tokens = query0.shape[0]
    query = query0.view(num_tokens, -1, head_size)
    key = key0.view(num_tokens, -1, head_size)
    cos, sin = cos_sin_cache[positions.long()].chunk(2, -1)
    cos = cos.repeat(1, 2).unsqueeze(-2)
    sin = sin.repeat(1, 2).unsqueeze(-2)

    def rotate(x):
        off = x.shape[2] // 2
        return torch.cat([-x[:, :, off:], x[:, :, :off]], -1)

    q_rot, k_rot = query[:, :, :rot_dim], key[:, :, :rot_dim]
    q_new = q_rot * cos + rotate(q_rot) * sin
    k_new = k_rot * cos + rotate(k_rot) * sin
    if head_size > rot_dim:
        q_new = torch.cat([q_new, query[:, :, rot_dim:]], -1)
        k_new = torch.cat([k_new, key[:, :, rot_dim:]], -1)
    query0.copy_(q_new.reshape(query0.shape))
    key0.copy_(k_new.reshape(key0.shape))


def make_cos_sin_cache(max_position, rot_dim, theta=10000.0, dtype=torch.bfloat16):
    """RotaryEmbedding::new, rllm-cuda/src/llm/mod.rs:41-60."""
    inv = 1.0 / (theta ** (torch.arange(0, rot_dim, 2, dtype=torch.float32) / rot_dim))
    idx = torch.arange(max_position, dtype=torch.float32).reshape(-1, 1) @ inv.reshape(1, -1)
    return torch.cat([idx.cos().to(dtype), idx.sin().to(dtype)], -1).contiguous()


def decode_step_cpu(query, key_cache, value_cache, num_kv_heads, scale, block_tables,
                    context_lens, block_size):
    """What rLLM's CPU build does for single-token sequences: there is no paged kernel
    (llm/config.rs:155-158), so each sequence goes gather_cached_kv -> repeat_kv ->
    varlen_attn with q_len = 1 (llm/mod.rs:168-278, 341-342).  fp32, as the CPU build runs
    (rllm-cuda.rs:37-39).  Returns [num_seqs, num_heads, head_size] fp32."""
    num_seqs, num_heads, head_size = query.shape
    ctx = context_lens.tolist()
    slots = []
    for s in range(num_seqs):
        bt = block_tables[s].tolist()
        slots += [bt[t // block_size] * block_size + t % block_size for t in range(ctx[s])]
    gather_mapping = torch.tensor(slots, dtype=torch.int32)
    k = torch.empty(len(slots), num_kv_heads, head_size, dtype=key_cache.dtype)
    v = torch.empty_like(k)
    gather_cached_kv(k, v, key_cache, value_cache, gather_mapping)
    n_rep = num_heads // num_kv_heads
    k, v = repeat_kv(k, n_rep), repeat_kv(v, n_rep)
    cu_q = torch.arange(num_seqs + 1, dtype=torch.int32)
    cu_k = torch.tensor([0] + ctx, dtype=torch.int64).cumsum(0).to(torch.int32)
    return varlen_attn(query, k, v, cu_q, cu_k, 1, max(ctx) if ctx else 0, scale, True)


def default_scale(head_dim):
    return 1.0 / math.sqrt(head_dim)
