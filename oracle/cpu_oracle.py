"""ctypes front-end of the C oracle (oracle/oracle.c) -- TEST INFRASTRUCTURE ONLY.

Functions take CPU torch tensors laid out exactly as the reference's kernels expect and
use the reference's own names (rllm/tch-cuda/src/lib.rs).  Nothing under ``aici_b200/``
imports this module; only tests, the smoke check and the benchmark's CPU-baseline leg do.
"""
import ctypes
import os

import numpy as np
import torch

from . import build_oracle

_lib = None


def lib():
    global _lib
    if _lib is None:
        path = build_oracle.OUT
        if not os.path.exists(path) or os.path.getmtime(path) < os.path.getmtime(build_oracle.SRC):
            path = build_oracle.build()
        _lib = ctypes.CDLL(path)
    return _lib


def _u16(t: torch.Tensor):
    assert t.device.type == "cpu" and t.dtype == torch.bfloat16
    return ctypes.c_void_p(t.data_ptr())


def _ptr(t: torch.Tensor):
    assert t.device.type == "cpu"
    return ctypes.c_void_p(t.data_ptr())


def reshape_and_cache(key, value, key_cache, value_cache, slot_mapping):
    """In place on key_cache/value_cache. cache_kernels.cu:168-253."""
    num_tokens, num_heads, head_size = key.shape
    block_size, x = key_cache.shape[3], key_cache.shape[4]
    assert key.stride(2) == 1 and key.stride(1) == head_size
    assert value.stride(2) == 1 and value.stride(1) == head_size
    assert key_cache.is_contiguous() and value_cache.is_contiguous()
    slots = slot_mapping.to(torch.int64).contiguous()
    lib().oracle_reshape_and_cache(
        _u16(key), _u16(value), _u16(key_cache), _u16(value_cache), _ptr(slots),
        ctypes.c_int(num_tokens), ctypes.c_int64(key.stride(0)), ctypes.c_int64(value.stride(0)),
        ctypes.c_int(num_heads), ctypes.c_int(head_size), ctypes.c_int(block_size), ctypes.c_int(x))


def gather_cached_kv(key, value, key_cache, value_cache, slot_mapping):
    """In place on key/value. cache_kernels.cu:301-413."""
    num_tokens, num_heads, head_size = key.shape
    block_size, x = key_cache.shape[3], key_cache.shape[4]
    assert key.stride(2) == 1 and key.stride(1) == head_size
    slots = slot_mapping.to(torch.int32).contiguous()
    lib().oracle_gather_cached_kv(
        _u16(key), _u16(value), _u16(key_cache), _u16(value_cache), _ptr(slots),
        ctypes.c_int(num_tokens), ctypes.c_int64(key.stride(0)), ctypes.c_int64(value.stride(0)),
        ctypes.c_int(num_heads), ctypes.c_int(head_size), ctypes.c_int(block_size), ctypes.c_int(x))


def copy_blocks(key_caches, value_caches, block_mapping):
    """block_mapping: dict src -> [dst...] as in lib.rs:276-280, or a flat list of pairs."""
    num_layers = len(key_caches)
    if num_layers == 0:
        return
    pairs = []
    if isinstance(block_mapping, dict):
        for src, dsts in block_mapping.items():
            for dst in dsts:
                pairs += [int(src), int(dst)]
    else:
        pairs = [int(v) for v in block_mapping]
    numel = key_caches[0][0].numel()
    kp = (ctypes.c_void_p * num_layers)(*[t.data_ptr() for t in key_caches])
    vp = (ctypes.c_void_p * num_layers)(*[t.data_ptr() for t in value_caches])
    mp = (ctypes.c_int64 * len(pairs))(*pairs)
    lib().oracle_copy_blocks(kp, vp, mp, ctypes.c_int(num_layers), ctypes.c_int(len(pairs) // 2),
                             ctypes.c_int64(numel))


def swap_blocks(src, dst, block_mapping):
    """dst[d] = src[s] for every s -> d, in ascending order of s as std::map iterates
    (cache_kernels.cu:12-50).  Both CPU tensors of shape [num_blocks, ...]."""
    pairs = sorted(block_mapping.items()) if isinstance(block_mapping, dict) else [
        (int(block_mapping[2 * i]), int(block_mapping[2 * i + 1]))
        for i in range(len(block_mapping) // 2)]
    for s, d in pairs:
        dst[d].copy_(src[s])


def _paged_common(query, key_cache, value_cache, block_tables, context_lens):
    num_seqs, num_heads, head_size = query.shape
    assert query.stride(2) == 1 and query.stride(1) == head_size
    block_size, x = key_cache.shape[3], key_cache.shape[4]
    bt = block_tables.to(torch.int32).contiguous()
    cl = context_lens.to(torch.int32).contiguous()
    out = torch.zeros(num_seqs, num_heads, head_size, dtype=torch.float32)
    return num_seqs, num_heads, head_size, block_size, x, bt, cl, out


def paged_attention_v1(query, key_cache, value_cache, num_kv_heads, scale, block_tables,
                       context_lens, ref_rounding=False):
    """Returns the fp32 result [num_seqs, num_heads, head_size]. attention_kernels.cu:85-418."""
    num_seqs, num_heads, head_size, block_size, x, bt, cl, out = _paged_common(
        query, key_cache, value_cache, block_tables, context_lens)
    lib().oracle_paged_attention_v1(
        _ptr(out), _u16(query), _u16(key_cache), _u16(value_cache), ctypes.c_int(num_kv_heads),
        ctypes.c_float(scale), _ptr(bt), _ptr(cl), ctypes.c_int(num_seqs), ctypes.c_int(num_heads),
        ctypes.c_int(head_size), ctypes.c_int(block_size), ctypes.c_int(x),
        ctypes.c_int(bt.shape[1] if bt.dim() == 2 else 0), ctypes.c_int64(query.stride(0)),
        ctypes.c_int64(key_cache.stride(0)), ctypes.c_int64(key_cache.stride(1)),
        ctypes.c_int(1 if ref_rounding else 0))
    return out


def paged_attention_v2(query, key_cache, value_cache, num_kv_heads, scale, block_tables,
                       context_lens, partition_size=512, ref_rounding=False):
    """Partitioned variant + reduce. attention_kernels.cu:421-546."""
    num_seqs, num_heads, head_size, block_size, x, bt, cl, out = _paged_common(
        query, key_cache, value_cache, block_tables, context_lens)
    lib().oracle_paged_attention_v2(
        _ptr(out), _u16(query), _u16(key_cache), _u16(value_cache), ctypes.c_int(num_kv_heads),
        ctypes.c_float(scale), _ptr(bt), _ptr(cl), ctypes.c_int(num_seqs), ctypes.c_int(num_heads),
        ctypes.c_int(head_size), ctypes.c_int(block_size), ctypes.c_int(x),
        ctypes.c_int(bt.shape[1] if bt.dim() == 2 else 0), ctypes.c_int64(query.stride(0)),
        ctypes.c_int64(key_cache.stride(0)), ctypes.c_int64(key_cache.stride(1)),
        ctypes.c_int(partition_size), ctypes.c_int(1 if ref_rounding else 0))
    return out


def _varlen_args(q, k, v):
    for t in (q, k, v):
        assert t.stride(2) == 1
    return [ctypes.c_int64(q.stride(0)), ctypes.c_int64(q.stride(1)),
            ctypes.c_int64(k.stride(0)), ctypes.c_int64(k.stride(1)),
            ctypes.c_int64(v.stride(0)), ctypes.c_int64(v.stride(1))]


def flash_attn_varlen(q, k, v, seqlens_q, seqlens_k, max_seqlen_q, max_seqlen_k,
                      softmax_scale, causal, p_bf16=False):
    """fp32 result [total_q, Hq, D]; argument list of lib.rs:69-79."""
    total_q, num_heads, head_size = q.shape
    num_heads_k = k.shape[1]
    cq = seqlens_q.to(torch.int32).contiguous()
    ck = seqlens_k.to(torch.int32).contiguous()
    out = torch.zeros(total_q, num_heads, head_size, dtype=torch.float32)
    lib().oracle_varlen_attn(
        _ptr(out), _u16(q), _u16(k), _u16(v), _ptr(cq), _ptr(ck), ctypes.c_int(cq.numel() - 1),
        ctypes.c_int(num_heads), ctypes.c_int(num_heads_k), ctypes.c_int(head_size),
        *_varlen_args(q, k, v), ctypes.c_float(softmax_scale), ctypes.c_int(1 if causal else 0),
        ctypes.c_int(1 if p_bf16 else 0))
    return out


def flash_attn_varlen_rows(q, k, v, seqlens_q, seqlens_k, rows, softmax_scale, causal,
                           p_bf16=False):
    """rows: int tensor [n, 3] of (seq, packed token index, head). Returns fp32 [n, D]."""
    num_heads, head_size = q.shape[1], q.shape[2]
    cq = seqlens_q.to(torch.int32).contiguous()
    ck = seqlens_k.to(torch.int32).contiguous()
    rows = rows.to(torch.int32)
    rs, rt, rh = (rows[:, i].contiguous() for i in range(3))
    out = torch.zeros(rows.shape[0], head_size, dtype=torch.float32)
    lib().oracle_varlen_attn_rows(
        _ptr(out), _u16(q), _u16(k), _u16(v), _ptr(cq), _ptr(ck), _ptr(rs), _ptr(rt), _ptr(rh),
        ctypes.c_int(rows.shape[0]), ctypes.c_int(num_heads), ctypes.c_int(k.shape[1]),
        ctypes.c_int(head_size), *_varlen_args(q, k, v), ctypes.c_float(softmax_scale),
        ctypes.c_int(1 if causal else 0), ctypes.c_int(1 if p_bf16 else 0))
    return out


def rotary_embedding(positions, query, key, head_size, cos_sin_cache, is_neox=True):
    """In place on query [T, Hq*D] / key [T, Hkv*D] (or 3-D). pos_encoding_kernels.cu:9-128."""
    assert is_neox, "the reference's CPU path implements only the NeoX pairing (refkernels.rs:170-185)"
    T = query.shape[0]
    q2, k2 = query.view(T, -1), key.view(T, -1)
    assert q2.stride(1) == 1 and k2.stride(1) == 1
    pos = positions.to(torch.int64).contiguous()
    cs = cos_sin_cache.contiguous()
    lib().oracle_rotary_embedding_neox(
        _ptr(pos), _u16(query), _u16(key), _u16(cs), ctypes.c_int(T), ctypes.c_int(q2.shape[1] // head_size),
        ctypes.c_int(k2.shape[1] // head_size), ctypes.c_int(head_size), ctypes.c_int(cs.shape[1]),
        ctypes.c_int64(q2.stride(0)), ctypes.c_int64(k2.stride(0)))


def round_to_bf16(x: torch.Tensor) -> torch.Tensor:
    x = x.contiguous().to(torch.float32)
    out = torch.empty(x.shape, dtype=torch.bfloat16)
    lib().oracle_round_to_bf16(_ptr(x), _ptr(out), ctypes.c_int64(x.numel()))
    return out


def error_stats(got: torch.Tensor, want_f32: torch.Tensor):
    """(max-abs, mean-abs) of got - want in fp32."""
    d = (got.to(torch.float32) - want_f32.to(torch.float32)).abs()
    if d.numel() == 0:
        return 0.0, 0.0
    return float(d.max()), float(d.mean())
