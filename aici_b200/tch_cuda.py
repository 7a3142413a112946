"""Host-side mirror of the `tch-cuda` crate's public functions for the attention path.

Same names, argument order and meaning as rllm/tch-cuda/src/lib.rs (flash_attn_varlen :69-104,
reshape_and_cache :192-213, gather_cached_kv :215-234, copy_blocks :276-331,
paged_attention_v1 :356-391) plus `paged_attention_v2`, for which the crate has only the
extern (:122-137).  Tensors are torch CUDA tensors; this module extracts pointers, sizes,
strides and the current stream and calls the C ABI (include/aici_b200.h).  All arithmetic
runs in libaici_b200.so; torch only owns the memory and the stream.

Errors: the crate panics with "<fn>: <message>"; here an `AiciError` carries the same text.
"""
import ctypes
from typing import Dict, List, Optional, Sequence

import torch

from . import _lib
from ._lib import AiciError

_DTYPES = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}

_workspaces: Dict[tuple, torch.Tensor] = {}


class _on_device:
    """Makes `dev` the current CUDA device for the duration of a call; does nothing (and costs
    next to nothing) when it already is, which is the case on every call of a one-GPU process."""
    __slots__ = ("index", "prev")

    def __init__(self, dev: torch.device):
        self.index = dev.index if dev.index is not None else torch.cuda.current_device()
        self.prev = -1

    def __enter__(self):
        cur = torch.cuda.current_device()
        if cur != self.index:
            self.prev = cur
            torch.cuda.set_device(self.index)
        return self

    def __exit__(self, *exc):
        if self.prev >= 0:
            torch.cuda.set_device(self.prev)
        return False


def _p(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _stream(dev: torch.device):
    return ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)


def _require_cuda(fn: str, *tensors: torch.Tensor):
    dev = tensors[0].device
    for t in tensors:
        if not t.is_cuda:
            raise AiciError("%s: tensor must be on a CUDA device (there is no CPU path)" % fn)
        if t.device != dev:
            raise AiciError("%s: tensors are on different devices" % fn)
    return dev


def _dtype(fn: str, t: torch.Tensor) -> int:
    if t.dtype not in _DTYPES:
        raise AiciError("%s: unsupported dtype %s" % (fn, t.dtype))
    return _DTYPES[t.dtype]


def _cache_dims(fn: str, key_cache: torch.Tensor, value_cache: torch.Tensor):
    if key_cache.dim() != 5 or value_cache.dim() != 4:
        raise AiciError("%s: key_cache must be 5-D and value_cache 4-D" % fn)
    num_blocks, num_kv_heads, hs_x, block_size, x = key_cache.shape
    if not key_cache.is_contiguous() or not value_cache.is_contiguous():
        raise AiciError("%s: caches must be contiguous" % fn)
    if tuple(value_cache.shape) != (num_blocks, num_kv_heads, hs_x * x, block_size):
        raise AiciError("%s: value_cache shape does not match key_cache" % fn)
    if x * key_cache.element_size() != 16:
        raise AiciError("%s: last key_cache dimension must span 16 bytes" % fn)
    return num_blocks, num_kv_heads, hs_x * x, block_size


def flash_attn_varlen(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, seqlens_q: torch.Tensor,
                      seqlens_k: torch.Tensor, max_seqlen_q: int, max_seqlen_k: int,
                      softmax_scale: float, causal: bool, shape: int = 0) -> torch.Tensor:
    """softmax(Q K^T * softmax_scale) V over packed variable-length sequences; returns a new
    tensor [total_q, num_heads_q, head_size] (lib.rs:49-104).  `seqlens_*` are the cumulative
    lengths, int32, batch + 1 entries.  `shape` (not in the crate; tests and benchmarks) forces one
    of the kernel's shapes, see aici_mha_varlen_fwd_shape; 0 lets the sequence length choose."""
    fn = "flash_attn_varlen"
    dev = _require_cuda(fn, q, k, v, seqlens_q, seqlens_k)
    if q.dim() != 3 or k.dim() != 3 or v.dim() != 3:
        raise AiciError("%s: q, k, v must be 3-D" % fn)
    if k.dtype != q.dtype:
        raise AiciError("%s: query and key must have the same dtype" % fn)
    if v.dtype != q.dtype:
        raise AiciError("%s: query and value must have the same dtype" % fn)
    if seqlens_q.dtype != torch.int32:
        raise AiciError("%s: cu_seqlens_q must have dtype int32" % fn)
    if seqlens_k.dtype != torch.int32:
        raise AiciError("%s: cu_seqlens_k must have dtype int32" % fn)
    for t in (q, k, v):
        if t.stride(-1) != 1:
            raise AiciError("%s: Input tensor must have contiguous last dimension" % fn)
    if not seqlens_q.is_contiguous() or not seqlens_k.is_contiguous():
        raise AiciError("%s: cu_seqlens must be contiguous" % fn)
    batch = seqlens_q.numel() - 1
    if seqlens_k.numel() != batch + 1:
        raise AiciError("%s: cu_seqlens_q and cu_seqlens_k differ in length" % fn)
    if batch <= 0:
        raise AiciError("%s: batch size must be positive" % fn)
    total_q, num_heads, head_size = q.shape
    total_k, num_heads_k, _ = k.shape
    if tuple(v.shape) != tuple(k.shape) or k.shape[2] != head_size:
        raise AiciError("%s: k and v must be [total_k, num_heads_k, head_size]" % fn)
    out = torch.empty((total_q, num_heads, head_size), dtype=q.dtype, device=dev)
    head = (_p(out), _p(q), _p(k), _p(v), _p(seqlens_q), _p(seqlens_k), ctypes.c_int(batch),
            ctypes.c_int(total_q), ctypes.c_int(total_k), ctypes.c_int(num_heads),
            ctypes.c_int(num_heads_k), ctypes.c_int(head_size), ctypes.c_int(int(max_seqlen_q)),
            ctypes.c_int(int(max_seqlen_k)),
            ctypes.c_int64(q.stride(0)), ctypes.c_int64(q.stride(1)),
            ctypes.c_int64(k.stride(0)), ctypes.c_int64(k.stride(1)),
            ctypes.c_int64(v.stride(0)), ctypes.c_int64(v.stride(1)),
            ctypes.c_int64(out.stride(0)), ctypes.c_int64(out.stride(1)),
            ctypes.c_float(softmax_scale), ctypes.c_int(1 if causal else 0))
    with _on_device(dev):
        if shape:
            res = _lib.lib().aici_mha_varlen_fwd_shape(*head, ctypes.c_int(int(shape)), ctypes.c_int(_dtype(fn, q)),
                                                       _stream(dev))
        else:
            res = _lib.lib().aici_mha_varlen_fwd(*head, ctypes.c_int(_dtype(fn, q)), _stream(dev))
    _lib.check(fn, res)
    return out


# rllm-cuda re-exports flash_attn_varlen under this name (rllm-cuda/src/llm/kernels.rs:4-7).
varlen_attn = flash_attn_varlen


def reshape_and_cache(key: torch.Tensor, value: torch.Tensor, key_cache: torch.Tensor,
                      value_cache: torch.Tensor, slot_mapping: torch.Tensor) -> None:
    """key/value [num_tokens, num_heads, head_size] -> paged caches at slot_mapping
    (lib.rs:192-213).  slot_mapping may be int32 (as rLLM builds it) or int64 (as the crate
    casts it); no cast kernel runs here."""
    fn = "reshape_and_cache"
    dev = _require_cuda(fn, key, value, key_cache, value_cache, slot_mapping)
    num_blocks, num_kv_heads, head_size, block_size = _cache_dims(fn, key_cache, value_cache)
    if key.dim() != 3 or tuple(key.shape) != tuple(value.shape):
        raise AiciError("%s: key and value must be [num_tokens, num_heads, head_size]" % fn)
    if key.shape[1] != num_kv_heads or key.shape[2] != head_size:
        raise AiciError("%s: key shape does not match the cache" % fn)
    if key.stride(2) != 1 or key.stride(1) != head_size or value.stride(2) != 1 or \
            value.stride(1) != head_size:
        raise AiciError("%s: heads of one token must be contiguous" % fn)
    if slot_mapping.dtype not in (torch.int32, torch.int64) or not slot_mapping.is_contiguous():
        raise AiciError("%s: slot_mapping must be contiguous int32 or int64" % fn)
    if slot_mapping.numel() != key.shape[0]:
        raise AiciError("%s: slot_mapping must have one entry per token" % fn)
    if key_cache.dtype != key.dtype or value_cache.dtype != key.dtype:
        raise AiciError("%s: cache dtype differs from key dtype" % fn)
    with _on_device(dev):
        res = _lib.lib().aici_reshape_and_cache(
            _p(key), _p(value), _p(key_cache), _p(value_cache), _p(slot_mapping),
            ctypes.c_int(1 if slot_mapping.dtype == torch.int64 else 0),
            ctypes.c_int(key.shape[0]), ctypes.c_int(num_kv_heads), ctypes.c_int(head_size),
            ctypes.c_int(block_size), ctypes.c_int64(num_blocks), ctypes.c_int64(key.stride(0)),
            ctypes.c_int64(value.stride(0)), ctypes.c_int(_dtype(fn, key)), _stream(dev))
    _lib.check(fn, res)


def gather_cached_kv(key: torch.Tensor, value: torch.Tensor, key_cache: torch.Tensor,
                     value_cache: torch.Tensor, slot_mapping: torch.Tensor) -> None:
    """Inverse of reshape_and_cache: fills key/value from the caches (lib.rs:215-234)."""
    fn = "gather_cached_kv"
    dev = _require_cuda(fn, key, value, key_cache, value_cache, slot_mapping)
    num_blocks, num_kv_heads, head_size, block_size = _cache_dims(fn, key_cache, value_cache)
    if key.dim() != 3 or tuple(key.shape) != tuple(value.shape):
        raise AiciError("%s: key and value must be [num_tokens, num_heads, head_size]" % fn)
    if key.shape[1] != num_kv_heads or key.shape[2] != head_size:
        raise AiciError("%s: key shape does not match the cache" % fn)
    if key.stride(2) != 1 or key.stride(1) != head_size or value.stride(2) != 1 or \
            value.stride(1) != head_size:
        raise AiciError("%s: heads of one token must be contiguous" % fn)
    if slot_mapping.dtype != torch.int32 or not slot_mapping.is_contiguous():
        raise AiciError("%s: slot_mapping must be contiguous int32" % fn)
    if slot_mapping.numel() != key.shape[0]:
        raise AiciError("%s: slot_mapping must have one entry per token" % fn)
    with _on_device(dev):
        res = _lib.lib().aici_gather_cached_kv(
            _p(key), _p(value), _p(key_cache), _p(value_cache), _p(slot_mapping),
            ctypes.c_int(key.shape[0]), ctypes.c_int(num_kv_heads), ctypes.c_int(head_size),
            ctypes.c_int(block_size), ctypes.c_int64(num_blocks), ctypes.c_int64(key.stride(0)),
            ctypes.c_int64(value.stride(0)), ctypes.c_int(_dtype(fn, key)), _stream(dev))
    _lib.check(fn, res)


def copy_blocks(key_caches: Sequence[torch.Tensor], value_caches: Sequence[torch.Tensor],
                block_mapping) -> None:
    """For every layer and every src -> dst in block_mapping (a dict src -> [dst, ...] as in the
    crate, or the same pairs already flattened into an int64 CPU tensor) copy one key block and
    one value block (lib.rs:276-331).  The layer addresses and the pairs go to the kernel as arguments
    from host memory, so nothing is uploaded and nothing synchronises."""
    fn = "copy_blocks"
    num_layers = len(key_caches)
    if num_layers != len(value_caches):
        raise AiciError("%s: key_caches and value_caches differ in length" % fn)
    if num_layers == 0:
        return
    dev = key_caches[0].device
    if not dev.type == "cuda":
        raise AiciError("%s: caches must be on a CUDA device (there is no CPU path)" % fn)
    tsize = key_caches[0].numel()
    for t in list(key_caches) + list(value_caches):
        if t.device != dev or t.numel() != tsize:
            raise AiciError("%s: all caches must share device and size" % fn)
        if t.dtype not in (torch.bfloat16, torch.float16) or not t.is_contiguous():
            raise AiciError("%s: caches must be contiguous bf16 or f16" % fn)
    num_blocks, num_heads, head_size, block_size = value_caches[0].shape
    numel_per_block = num_heads * head_size * block_size
    if isinstance(block_mapping, torch.Tensor):
        # already flattened (src, dst, src, dst, ...) int64 host tensor: no per-pair Python work
        if block_mapping.dtype != torch.int64 or block_mapping.is_cuda or not block_mapping.is_contiguous():
            raise AiciError("%s: a flattened block_mapping must be a contiguous int64 CPU tensor" % fn)
        flat = block_mapping
    else:
        pairs: List[int] = []
        for src, dsts in block_mapping.items():
            for dst in dsts:
                pairs += [int(src), int(dst)]
        flat = torch.tensor(pairs, dtype=torch.int64)
    num_pairs = flat.numel() // 2
    if num_pairs == 0:
        return
    kp = (ctypes.c_int64 * num_layers)(*[t.data_ptr() for t in key_caches])
    vp = (ctypes.c_int64 * num_layers)(*[t.data_ptr() for t in value_caches])
    mp = ctypes.c_void_p(flat.data_ptr())
    with _on_device(dev):
        res = _lib.lib().aici_copy_blocks_host(
            kp, vp, mp, ctypes.c_int(num_layers), ctypes.c_int(num_pairs),
            ctypes.c_int64(numel_per_block), ctypes.c_int64(num_blocks),
            ctypes.c_int(_dtype(fn, key_caches[0])), _stream(dev))
    _lib.check(fn, res)


def copy_blocks_2(key_cache_ptrs_tensor: torch.Tensor, value_cache_ptrs_tensor: torch.Tensor,
                  block_mapping_tensor: torch.Tensor, key0: torch.Tensor) -> None:
    """The extern's own calling convention (lib.rs:184-189): three int64 device tensors plus
    the first key cache, from which block size and dtype are read."""
    fn = "copy_blocks_2"
    dev = _require_cuda(fn, key_cache_ptrs_tensor, value_cache_ptrs_tensor, block_mapping_tensor, key0)
    for t in (key_cache_ptrs_tensor, value_cache_ptrs_tensor, block_mapping_tensor):
        if t.dtype != torch.int64 or not t.is_contiguous():
            raise AiciError("%s: pointer and mapping tensors must be contiguous int64" % fn)
    num_layers = key_cache_ptrs_tensor.numel()
    num_pairs = block_mapping_tensor.numel() // 2
    with _on_device(dev):
        res = _lib.lib().aici_copy_blocks(
            _p(key_cache_ptrs_tensor), _p(value_cache_ptrs_tensor), _p(block_mapping_tensor),
            ctypes.c_int(num_layers), ctypes.c_int(num_pairs), ctypes.c_int64(key0[0].numel()),
            ctypes.c_int64(key0.shape[0]), ctypes.c_int(_dtype(fn, key0)), _stream(dev))
    _lib.check(fn, res)


def swap_blocks(src: torch.Tensor, dst: torch.Tensor, block_mapping) -> None:
    """`kernels::swap_blocks(src, dst, src_to_dst, stream)` as CacheEngine::swap calls it per layer
    for K and for V (rllm-cuda/src/llm/paged/cache_engine.rs:139-149; C side
    kernels/vllm/cache_kernels.cu:12-50): dst[d] = src[s] for every s -> d of `block_mapping`
    (dict, or a flat int64 CPU tensor of (src, dst) pairs).  Either tensor may live in host memory
    (page-locked: one kernel launch over PCIe; pageable: copy engine); at least one is on the GPU.
    Runs on the current stream of the CUDA tensor's device."""
    fn = "swap_blocks"
    if src.dim() < 1 or dst.dim() < 1 or src.shape[1:] != dst.shape[1:] or src.dtype != dst.dtype:
        raise AiciError("%s: src and dst must have the same block shape and dtype" % fn)
    if not src.is_contiguous() or not dst.is_contiguous():
        raise AiciError("%s: caches must be contiguous" % fn)
    cuda = [t for t in (src, dst) if t.is_cuda]
    if not cuda:
        raise AiciError("%s: Invalid device combination" % fn)
    if len(cuda) == 2 and src.device != dst.device:
        raise AiciError("%s: src and dst must be on the same GPU" % fn)
    if isinstance(block_mapping, torch.Tensor):
        pairs = block_mapping.to(torch.int64).contiguous().view(-1)
        if pairs.is_cuda:
            raise AiciError("%s: block_mapping must be a CPU tensor" % fn)
    else:
        flat: List[int] = []
        for s, d in block_mapping.items():
            flat += [int(s), int(d)]
        pairs = torch.tensor(flat, dtype=torch.int64)
    if pairs.numel() == 0:
        return
    dev = cuda[0].device
    block_bytes = src[0].numel() * src.element_size()
    with _on_device(dev):
        _lib.check(fn, _lib.lib().aici_swap_blocks(
            _p(src), _p(dst), ctypes.c_void_p(pairs.data_ptr()), ctypes.c_int(pairs.numel() // 2),
            ctypes.c_int64(block_bytes), ctypes.c_int64(src.shape[0]), ctypes.c_int64(dst.shape[0]),
            _stream(dev)))


def _decode_common(fn, out, query, key_cache, value_cache, num_kv_heads, block_tables,
                   context_lens, block_size):
    dev = _require_cuda(fn, out, query, key_cache, value_cache, block_tables, context_lens)
    num_blocks, cache_kv_heads, head_size, cache_block = _cache_dims(fn, key_cache, value_cache)
    if cache_kv_heads != num_kv_heads:
        raise AiciError("%s: num_kv_heads does not match the cache" % fn)
    if cache_block != block_size:
        raise AiciError("%s: block_size does not match the cache" % fn)
    if query.dim() != 3 or tuple(out.shape) != tuple(query.shape):
        raise AiciError("%s: out and query must be [num_seqs, num_heads, head_size]" % fn)
    if query.shape[2] != head_size or query.stride(2) != 1 or query.stride(1) != head_size:
        raise AiciError("%s: query rows must hold contiguous heads of the cache's head_size" % fn)
    if not out.is_contiguous():
        raise AiciError("%s: out must be contiguous" % fn)
    if block_tables.dtype != torch.int32 or context_lens.dtype != torch.int32:
        raise AiciError("%s: block_tables and context_lens must be int32" % fn)
    if not block_tables.is_contiguous() or not context_lens.is_contiguous():
        raise AiciError("%s: block_tables and context_lens must be contiguous" % fn)
    if block_tables.dim() != 2 or block_tables.shape[0] != query.shape[0] or \
            context_lens.numel() != query.shape[0]:
        raise AiciError("%s: block_tables must be [num_seqs, max_blocks], context_lens [num_seqs]" % fn)
    if query.dtype != key_cache.dtype or out.dtype != query.dtype:
        raise AiciError("%s: dtypes differ" % fn)
    return dev, num_blocks, head_size


def _workspace(dev: torch.device, nbytes: int) -> torch.Tensor:
    """Scratch for the split-context partials; cached per (device, stream) and grown on
    demand (one inference thread owns a stream, rllm-base/src/server/mod.rs:470-502)."""
    key = (dev.index, torch.cuda.current_stream(dev).cuda_stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        _workspaces[key] = ws
    return ws


def paged_attention_v1(out: torch.Tensor, query: torch.Tensor, key_cache: torch.Tensor,
                       value_cache: torch.Tensor, num_kv_heads: int, scale: float,
                       block_tables: torch.Tensor, context_lens: torch.Tensor, block_size: int,
                       max_context_len: int, alibi_slopes: Optional[torch.Tensor]) -> None:
    """Decode attention for one query token per sequence over the paged cache, written into
    `out` (lib.rs:356-391)."""
    fn = "paged_attention_v1"
    if alibi_slopes is not None:
        raise AiciError("%s: alibi_slopes is not supported" % fn)
    dev, num_blocks, head_size = _decode_common(fn, out, query, key_cache, value_cache,
                                                num_kv_heads, block_tables, context_lens, block_size)
    num_seqs, num_heads, _ = query.shape
    L = _lib.lib()
    with _on_device(dev):
        nbytes = L.aici_paged_attention_workspace_bytes(
            ctypes.c_int(num_seqs), ctypes.c_int(num_heads), ctypes.c_int(num_kv_heads),
            ctypes.c_int(int(max_context_len)))
        ws = _workspace(dev, nbytes)
        res = L.aici_paged_attention_v1(
            _p(out), _p(query), _p(key_cache), _p(value_cache), ctypes.c_int(num_kv_heads),
            ctypes.c_float(scale), _p(block_tables), _p(context_lens), ctypes.c_int(block_size),
            ctypes.c_int(int(max_context_len)), ctypes.c_void_p(0), ctypes.c_int(num_seqs),
            ctypes.c_int(num_heads), ctypes.c_int(head_size), ctypes.c_int(block_tables.shape[1]),
            ctypes.c_int64(num_blocks), ctypes.c_int64(query.stride(0)),
            ctypes.c_int64(key_cache.stride(0)), ctypes.c_int64(key_cache.stride(1)),
            _p(ws), ctypes.c_size_t(ws.numel()), ctypes.c_int(_dtype(fn, query)), _stream(dev))
    _lib.check(fn, res)


def paged_attention_v1_chunked(out: torch.Tensor, query: torch.Tensor, key_cache: torch.Tensor,
                               value_cache: torch.Tensor, num_kv_heads: int, scale: float,
                               block_tables: torch.Tensor, context_lens: torch.Tensor, block_size: int,
                               max_context_len: int, chunk_tokens: int) -> None:
    """paged_attention_v1 through the fixed-chunk traversal with `chunk_tokens` tokens per chunk (0 =
    the library's choice).  Test and benchmark hook: results match paged_attention_v1 up to the
    rounding of different split points."""
    fn = "paged_attention_v1_chunked"
    dev, num_blocks, head_size = _decode_common(fn, out, query, key_cache, value_cache,
                                                num_kv_heads, block_tables, context_lens, block_size)
    num_seqs, num_heads, _ = query.shape
    L = _lib.lib()
    with _on_device(dev):
        nbytes = L.aici_paged_attention_chunked_workspace_bytes(
            ctypes.c_int(num_seqs), ctypes.c_int(num_heads), ctypes.c_int(num_kv_heads),
            ctypes.c_int(int(max_context_len)), ctypes.c_int(int(chunk_tokens)))
        ws = _workspace(dev, nbytes)
        res = L.aici_paged_attention_v1_chunked(
            _p(out), _p(query), _p(key_cache), _p(value_cache), ctypes.c_int(num_kv_heads),
            ctypes.c_float(scale), _p(block_tables), _p(context_lens), ctypes.c_int(block_size),
            ctypes.c_int(int(max_context_len)), ctypes.c_void_p(0), ctypes.c_int(num_seqs),
            ctypes.c_int(num_heads), ctypes.c_int(head_size), ctypes.c_int(block_tables.shape[1]),
            ctypes.c_int64(num_blocks), ctypes.c_int64(query.stride(0)),
            ctypes.c_int64(key_cache.stride(0)), ctypes.c_int64(key_cache.stride(1)),
            _p(ws), ctypes.c_size_t(ws.numel()), ctypes.c_int(int(chunk_tokens)),
            ctypes.c_int(_dtype(fn, query)), _stream(dev))
    _lib.check(fn, res)


def paged_attention_v2(out: torch.Tensor, exp_sums: torch.Tensor, max_logits: torch.Tensor,
                       tmp_out: torch.Tensor, query: torch.Tensor, key_cache: torch.Tensor,
                       value_cache: torch.Tensor, num_kv_heads: int, scale: float,
                       block_tables: torch.Tensor, context_lens: torch.Tensor, block_size: int,
                       max_context_len: int, alibi_slopes: Optional[torch.Tensor]) -> None:
    """Partitioned decode attention with caller-owned temporaries, argument list of the
    crate's extern (lib.rs:122-137): exp_sums/max_logits fp32 [num_seqs, num_heads, P],
    tmp_out [num_seqs, num_heads, P, head_size], P = ceil(max_context_len / 512)."""
    fn = "paged_attention_v2"
    if alibi_slopes is not None:
        raise AiciError("%s: alibi_slopes is not supported" % fn)
    dev, num_blocks, head_size = _decode_common(fn, out, query, key_cache, value_cache,
                                                num_kv_heads, block_tables, context_lens, block_size)
    num_seqs, num_heads, _ = query.shape
    parts = max(1, (int(max_context_len) + 511) // 512)
    _require_cuda(fn, out, exp_sums, max_logits, tmp_out)
    if exp_sums.dtype != torch.float32 or max_logits.dtype != torch.float32:
        raise AiciError("%s: exp_sums and max_logits must be float32" % fn)
    if tuple(exp_sums.shape) != (num_seqs, num_heads, parts) or \
            tuple(max_logits.shape) != (num_seqs, num_heads, parts) or \
            tuple(tmp_out.shape) != (num_seqs, num_heads, parts, head_size):
        raise AiciError("%s: temporaries must be sized for %d partitions" % (fn, parts))
    if not (exp_sums.is_contiguous() and max_logits.is_contiguous() and tmp_out.is_contiguous()):
        raise AiciError("%s: temporaries must be contiguous" % fn)
    if tmp_out.dtype != query.dtype:
        raise AiciError("%s: tmp_out dtype differs from query" % fn)
    with _on_device(dev):
        res = _lib.lib().aici_paged_attention_v2(
            _p(out), _p(exp_sums), _p(max_logits), _p(tmp_out), _p(query), _p(key_cache),
            _p(value_cache), ctypes.c_int(num_kv_heads), ctypes.c_float(scale), _p(block_tables),
            _p(context_lens), ctypes.c_int(block_size), ctypes.c_int(int(max_context_len)),
            ctypes.c_void_p(0), ctypes.c_int(num_seqs), ctypes.c_int(num_heads),
            ctypes.c_int(head_size), ctypes.c_int(block_tables.shape[1]), ctypes.c_int64(num_blocks),
            ctypes.c_int64(query.stride(0)), ctypes.c_int64(key_cache.stride(0)),
            ctypes.c_int64(key_cache.stride(1)), ctypes.c_int(_dtype(fn, query)), _stream(dev))
    _lib.check(fn, res)


def paged_attention_v1_static(out: torch.Tensor, query: torch.Tensor, key_cache: torch.Tensor,
                              value_cache: torch.Tensor, num_kv_heads: int, scale: float,
                              block_tables: torch.Tensor, context_lens: torch.Tensor, block_size: int,
                              max_context_len: int, alibi_slopes: Optional[torch.Tensor]) -> None:
    """paged_attention_v1 for callers that must not allocate at call time: no workspace tensor is
    created here and the library allocates nothing; the scratch is a 32 MiB array inside the
    library.  Larger batches raise.  Calls on one device must not overlap (keep one stream)."""
    fn = "paged_attention_v1_static"
    if alibi_slopes is not None:
        raise AiciError("%s: alibi_slopes is not supported" % fn)
    dev, num_blocks, head_size = _decode_common(fn, out, query, key_cache, value_cache,
                                                num_kv_heads, block_tables, context_lens, block_size)
    num_seqs, num_heads, _ = query.shape
    with _on_device(dev):
        res = _lib.lib().aici_paged_attention_v1_static(
            _p(out), _p(query), _p(key_cache), _p(value_cache), ctypes.c_int(num_kv_heads),
            ctypes.c_float(scale), _p(block_tables), _p(context_lens), ctypes.c_int(block_size),
            ctypes.c_int(int(max_context_len)), ctypes.c_void_p(0), ctypes.c_int(num_seqs),
            ctypes.c_int(num_heads), ctypes.c_int(head_size), ctypes.c_int(block_tables.shape[1]),
            ctypes.c_int64(num_blocks), ctypes.c_int64(query.stride(0)),
            ctypes.c_int64(key_cache.stride(0)), ctypes.c_int64(key_cache.stride(1)),
            ctypes.c_int(_dtype(fn, query)), _stream(dev))
    _lib.check(fn, res)


def flash_attn_varlen_paged(q: torch.Tensor, key_cache: torch.Tensor, value_cache: torch.Tensor,
                            seqlens_q: torch.Tensor, context_lens: torch.Tensor,
                            block_tables: torch.Tensor, max_seqlen_q: int, max_context_len: int,
                            softmax_scale: float, causal: bool) -> torch.Tensor:
    """Prefill attention with keys/values read from the paged cache through block tables: what
    compute_varlen_attn (rllm-cuda/src/llm/mod.rs:168-278) gets from gather_cached_kv + repeat_kv +
    flash_attn_varlen, without the gathered copy.  `seqlens_q` cumulative int32 [batch + 1];
    `context_lens` int32 [batch] (tokens of each sequence in the cache, new ones included);
    `block_tables` int32 [batch, max_blocks].  Returns [total_q, num_heads, head_size]."""
    fn = "flash_attn_varlen_paged"
    dev = _require_cuda(fn, q, key_cache, value_cache, seqlens_q, context_lens, block_tables)
    num_blocks, num_kv_heads, head_size, block_size = _cache_dims(fn, key_cache, value_cache)
    if q.dim() != 3 or q.shape[2] != head_size or q.stride(2) != 1:
        raise AiciError("%s: q must be [total_q, num_heads, head_size] with contiguous last dimension" % fn)
    for t in (seqlens_q, context_lens, block_tables):
        if t.dtype != torch.int32 or not t.is_contiguous():
            raise AiciError("%s: seqlens_q, context_lens and block_tables must be contiguous int32" % fn)
    batch = seqlens_q.numel() - 1
    if batch <= 0:
        raise AiciError("%s: batch size must be positive" % fn)
    if context_lens.numel() != batch or block_tables.dim() != 2 or block_tables.shape[0] != batch:
        raise AiciError("%s: context_lens must be [batch] and block_tables [batch, max_blocks]" % fn)
    if q.dtype != key_cache.dtype:
        raise AiciError("%s: query and cache dtypes differ" % fn)
    total_q, num_heads, _ = q.shape
    out = torch.empty((total_q, num_heads, head_size), dtype=q.dtype, device=dev)
    with _on_device(dev):
        res = _lib.lib().aici_mha_varlen_paged_fwd(
            _p(out), _p(q), _p(key_cache), _p(value_cache), _p(seqlens_q), _p(context_lens),
            _p(block_tables), ctypes.c_int(batch), ctypes.c_int(total_q), ctypes.c_int(num_heads),
            ctypes.c_int(num_kv_heads), ctypes.c_int(head_size), ctypes.c_int(block_size),
            ctypes.c_int(int(max_seqlen_q)), ctypes.c_int(int(max_context_len)),
            ctypes.c_int(block_tables.shape[1]), ctypes.c_int64(num_blocks),
            ctypes.c_int64(q.stride(0)), ctypes.c_int64(q.stride(1)),
            ctypes.c_int64(out.stride(0)), ctypes.c_int64(out.stride(1)),
            ctypes.c_int64(key_cache.stride(0)), ctypes.c_int64(key_cache.stride(1)),
            ctypes.c_float(softmax_scale), ctypes.c_int(1 if causal else 0),
            ctypes.c_int(_dtype(fn, q)), _stream(dev))
    _lib.check(fn, res)
    return out


def rotary_embedding_reshape_and_cache(positions: torch.Tensor, query: torch.Tensor, key: torch.Tensor,
                                       value: torch.Tensor, head_size: int, cos_sin_cache: torch.Tensor,
                                       is_neox: bool, key_cache: torch.Tensor, value_cache: torch.Tensor,
                                       slot_mapping: torch.Tensor) -> None:
    """rotary_embedding (lib.rs:333-354) and reshape_and_cache (lib.rs:192-213) in one pass:
    `query` [num_tokens, num_heads * head_size] and `key` [num_tokens, num_kv_heads * head_size]
    are rotated in place and the rotated key plus `value` go into the paged cache."""
    fn = "rotary_embedding_reshape_and_cache"
    dev = _require_cuda(fn, positions, query, key, value, cos_sin_cache, key_cache, value_cache, slot_mapping)
    num_blocks, num_kv_heads, cache_head, block_size = _cache_dims(fn, key_cache, value_cache)
    if cache_head != head_size:
        raise AiciError("%s: head_size does not match the cache" % fn)
    T = query.shape[0]
    q2, k2, v2 = query.view(T, -1), key.view(T, -1), value.view(T, -1)
    if q2.stride(1) != 1 or k2.stride(1) != 1 or v2.stride(1) != 1:
        raise AiciError("%s: rows must be contiguous" % fn)
    if k2.shape[1] != num_kv_heads * head_size or v2.shape[1] != k2.shape[1] or q2.shape[1] % head_size:
        raise AiciError("%s: key/value width does not match the cache" % fn)
    if positions.dtype != torch.int64 or not positions.is_contiguous() or positions.numel() != T:
        raise AiciError("%s: positions must be contiguous int64 [num_tokens]" % fn)
    if slot_mapping.dtype not in (torch.int32, torch.int64) or not slot_mapping.is_contiguous() or \
            slot_mapping.numel() != T:
        raise AiciError("%s: slot_mapping must be contiguous int32 or int64 [num_tokens]" % fn)
    if cos_sin_cache.dim() != 2 or not cos_sin_cache.is_contiguous() or cos_sin_cache.dtype != query.dtype:
        raise AiciError("%s: cos_sin_cache must be contiguous [max_position, rot_dim] of the query dtype" % fn)
    with _on_device(dev):
        res = _lib.lib().aici_rotary_reshape_and_cache(
            _p(positions), _p(query), _p(key), _p(value), _p(cos_sin_cache), _p(key_cache), _p(value_cache),
            _p(slot_mapping), ctypes.c_int(1 if slot_mapping.dtype == torch.int64 else 0), ctypes.c_int(T),
            ctypes.c_int(q2.shape[1] // head_size), ctypes.c_int(num_kv_heads), ctypes.c_int(head_size),
            ctypes.c_int(cos_sin_cache.shape[1]), ctypes.c_int(1 if is_neox else 0),
            ctypes.c_int64(cos_sin_cache.shape[0]), ctypes.c_int(block_size), ctypes.c_int64(num_blocks),
            ctypes.c_int64(q2.stride(0)), ctypes.c_int64(k2.stride(0)), ctypes.c_int64(v2.stride(0)),
            ctypes.c_int(_dtype(fn, query)), _stream(dev))
    _lib.check(fn, res)


def paged_attention_v1_peers(peer_ptrs: Sequence[int], total_heads: int, head0: int, query: torch.Tensor,
                             key_cache: torch.Tensor, value_cache: torch.Tensor, num_kv_heads: int,
                             scale: float, block_tables: torch.Tensor, context_lens: torch.Tensor,
                             block_size: int, max_context_len: int,
                             barrier_flags: Optional[Sequence[int]] = None, rank: int = 0) -> None:
    """paged_attention_v1 whose output rows go to head index head0 + h of the
    [num_seqs, total_heads, head_size] buffers at `peer_ptrs` (one device pointer per rank, this
    rank's own included; see aici_b200.sharding.PeerGather).  No collective follows; ranks
    synchronise before reading -- with a barrier of their own, or, when `barrier_flags` (the ranks'
    flag arrays) and `rank` are given, inside this call's last kernel."""
    fn = "paged_attention_v1_peers"
    dev = _require_cuda(fn, query, key_cache, value_cache, block_tables, context_lens)
    num_blocks, cache_kv_heads, head_size, cache_block = _cache_dims(fn, key_cache, value_cache)
    if cache_kv_heads != num_kv_heads or cache_block != block_size:
        raise AiciError("%s: num_kv_heads / block_size do not match the cache" % fn)
    if query.dim() != 3 or query.shape[2] != head_size or query.stride(2) != 1 or query.stride(1) != head_size:
        raise AiciError("%s: query rows must hold contiguous heads of the cache's head_size" % fn)
    if block_tables.dtype != torch.int32 or context_lens.dtype != torch.int32 or \
            not block_tables.is_contiguous() or not context_lens.is_contiguous():
        raise AiciError("%s: block_tables and context_lens must be contiguous int32" % fn)
    num_seqs, num_heads, _ = query.shape
    world = len(peer_ptrs)
    outs = (ctypes.c_void_p * world)(*[ctypes.c_void_p(int(x)) for x in peer_ptrs])
    L = _lib.lib()
    with _on_device(dev):
        nbytes = L.aici_paged_attention_workspace_bytes(
            ctypes.c_int(num_seqs), ctypes.c_int(num_heads), ctypes.c_int(num_kv_heads),
            ctypes.c_int(int(max_context_len)))
        ws = _workspace(dev, nbytes)
        tail = (_p(query), _p(key_cache), _p(value_cache), ctypes.c_int(num_kv_heads), ctypes.c_float(scale),
                _p(block_tables), _p(context_lens), ctypes.c_int(block_size), ctypes.c_int(int(max_context_len)),
                ctypes.c_int(num_seqs), ctypes.c_int(num_heads), ctypes.c_int(head_size),
                ctypes.c_int(block_tables.shape[1]), ctypes.c_int64(num_blocks), ctypes.c_int64(query.stride(0)),
                ctypes.c_int64(key_cache.stride(0)), ctypes.c_int64(key_cache.stride(1)), _p(ws),
                ctypes.c_size_t(ws.numel()), ctypes.c_int(_dtype(fn, query)), _stream(dev))
        if barrier_flags is None:
            res = L.aici_paged_attention_v1_peers(outs, ctypes.c_int(world), ctypes.c_int(total_heads),
                                                  ctypes.c_int(head0), *tail)
        else:
            if len(barrier_flags) != world:
                raise AiciError("%s: one flag array per rank is needed" % fn)
            flags = (ctypes.c_void_p * world)(*[ctypes.c_void_p(int(x)) for x in barrier_flags])
            res = L.aici_paged_attention_v1_peers_barrier(outs, flags, ctypes.c_int(world), ctypes.c_int(rank),
                                                          ctypes.c_int(total_heads), ctypes.c_int(head0), *tail)
    _lib.check(fn, res)


def decode_step(out: Optional[torch.Tensor], new_key: torch.Tensor, new_value: torch.Tensor,
                slot_mapping: torch.Tensor, query: torch.Tensor, key_cache: torch.Tensor,
                value_cache: torch.Tensor, num_kv_heads: int, scale: float, block_tables: torch.Tensor,
                context_lens: torch.Tensor, block_size: int, max_context_len: int,
                peer_ptrs: Optional[Sequence[int]] = None, barrier_flags: Optional[Sequence[int]] = None,
                rank: int = 0, total_heads: int = 0, head0: int = 0) -> None:
    """reshape_and_cache(new_key, new_value, ..., slot_mapping) followed by paged_attention_v1 into
    `out`, as one call (aici_decode_step): token i must be the newest token of sequence i
    (slot_mapping[i] = the cache slot of position context_lens[i] - 1); the library then lets the
    decode kernel read the rest of the cache while the write is still running.  With `peer_ptrs` /
    `barrier_flags` the output rows go to every rank's buffer instead of `out` and the call ends with
    the ranks' barrier (see paged_attention_v1_peers)."""
    fn = "decode_step"
    dev = _require_cuda(fn, new_key, new_value, slot_mapping, query, key_cache, value_cache, block_tables,
                        context_lens)
    num_blocks, cache_kv_heads, head_size, cache_block = _cache_dims(fn, key_cache, value_cache)
    if cache_kv_heads != num_kv_heads or cache_block != block_size:
        raise AiciError("%s: num_kv_heads / block_size do not match the cache" % fn)
    if query.dim() != 3 or query.shape[2] != head_size or query.stride(2) != 1 or query.stride(1) != head_size:
        raise AiciError("%s: query rows must hold contiguous heads of the cache's head_size" % fn)
    num_seqs, num_heads, _ = query.shape
    if tuple(new_key.shape) != (num_seqs, num_kv_heads, head_size) or tuple(new_value.shape) != tuple(new_key.shape):
        raise AiciError("%s: new key/value must be [num_seqs, num_kv_heads, head_size]" % fn)
    if new_key.stride(2) != 1 or new_key.stride(1) != head_size or new_value.stride(2) != 1 or \
            new_value.stride(1) != head_size:
        raise AiciError("%s: heads of one token must be contiguous" % fn)
    if slot_mapping.dtype not in (torch.int32, torch.int64) or not slot_mapping.is_contiguous() or \
            slot_mapping.numel() != num_seqs:
        raise AiciError("%s: slot_mapping must be contiguous int32 or int64 with one entry per sequence" % fn)
    if block_tables.dtype != torch.int32 or context_lens.dtype != torch.int32 or \
            not block_tables.is_contiguous() or not context_lens.is_contiguous():
        raise AiciError("%s: block_tables and context_lens must be contiguous int32" % fn)
    if peer_ptrs is None:
        if out is None or tuple(out.shape) != tuple(query.shape) or not out.is_contiguous() or out.device != dev:
            raise AiciError("%s: out must be a contiguous tensor shaped like query" % fn)
        ptrs, world, flags = [out.data_ptr()], 1, None
        total_heads, head0 = num_heads, 0
    else:
        ptrs, world = [int(x) for x in peer_ptrs], len(peer_ptrs)
        if world > 1 and (barrier_flags is None or len(barrier_flags) != world):
            raise AiciError("%s: one flag array per rank is needed" % fn)
        flags = barrier_flags
    outs = (ctypes.c_void_p * world)(*[ctypes.c_void_p(x) for x in ptrs])
    flag_arr = (ctypes.c_void_p * world)(*[ctypes.c_void_p(int(x)) for x in flags]) if flags is not None else None
    L = _lib.lib()
    with _on_device(dev):
        nbytes = L.aici_paged_attention_workspace_bytes(
            ctypes.c_int(num_seqs), ctypes.c_int(num_heads), ctypes.c_int(num_kv_heads),
            ctypes.c_int(int(max_context_len)))
        ws = _workspace(dev, nbytes)
        res = L.aici_decode_step(
            outs, flag_arr, ctypes.c_int(world), ctypes.c_int(rank), ctypes.c_int(total_heads), ctypes.c_int(head0),
            _p(new_key), _p(new_value), _p(slot_mapping), ctypes.c_int(1 if slot_mapping.dtype == torch.int64 else 0),
            ctypes.c_int64(new_key.stride(0)), ctypes.c_int64(new_value.stride(0)), _p(query), _p(key_cache),
            _p(value_cache), ctypes.c_int(num_kv_heads), ctypes.c_float(scale), _p(block_tables), _p(context_lens),
            ctypes.c_int(block_size), ctypes.c_int(int(max_context_len)), ctypes.c_int(num_seqs),
            ctypes.c_int(num_heads), ctypes.c_int(head_size), ctypes.c_int(block_tables.shape[1]),
            ctypes.c_int64(num_blocks), ctypes.c_int64(query.stride(0)), ctypes.c_int64(key_cache.stride(0)),
            ctypes.c_int64(key_cache.stride(1)), _p(ws), ctypes.c_size_t(ws.numel()),
            ctypes.c_int(_dtype(fn, query)), _stream(dev))
    _lib.check(fn, res)


def gather_heads(peer_ptrs: Sequence[int], total_heads: int, head0: int, local: torch.Tensor) -> None:
    """Stores local [rows, heads, 128] at head index head0 + h of every rank's
    [rows, total_heads, 128] buffer in `peer_ptrs` (the head-output gather as a call of its own; a
    barrier between the ranks has to follow before anyone reads)."""
    fn = "gather_heads"
    dev = _require_cuda(fn, local)
    if local.dim() != 3 or local.stride(2) != 1 or local.stride(1) != local.shape[2]:
        raise AiciError("%s: local must be [rows, heads, head_size] with contiguous heads" % fn)
    world = len(peer_ptrs)
    outs = (ctypes.c_void_p * world)(*[ctypes.c_void_p(int(x)) for x in peer_ptrs])
    with _on_device(dev):
        res = _lib.lib().aici_gather_heads(
            outs, ctypes.c_int(world), ctypes.c_int(total_heads), ctypes.c_int(head0), _p(local),
            ctypes.c_int64(local.shape[0]), ctypes.c_int(local.shape[1]), ctypes.c_int(local.shape[2]),
            ctypes.c_int64(local.stride(0)), ctypes.c_int(_dtype(fn, local)), _stream(dev))
    _lib.check(fn, res)


def flash_attn_varlen_peers(peer_ptrs: Sequence[int], total_heads: int, head0: int, q: torch.Tensor,
                            k: torch.Tensor, v: torch.Tensor, seqlens_q: torch.Tensor,
                            seqlens_k: torch.Tensor, max_seqlen_q: int, max_seqlen_k: int,
                            softmax_scale: float, causal: bool) -> None:
    """flash_attn_varlen whose output tiles go to head index head0 + h of the contiguous
    [total_q, total_heads, head_size] buffers at `peer_ptrs` (one per rank, own included)."""
    fn = "flash_attn_varlen_peers"
    dev = _require_cuda(fn, q, k, v, seqlens_q, seqlens_k)
    if seqlens_q.dtype != torch.int32 or seqlens_k.dtype != torch.int32:
        raise AiciError("%s: cu_seqlens must have dtype int32" % fn)
    for t in (q, k, v):
        if t.dim() != 3 or t.stride(-1) != 1:
            raise AiciError("%s: q, k, v must be 3-D with contiguous last dimension" % fn)
    total_q, num_heads, head_size = q.shape
    batch = seqlens_q.numel() - 1
    world = len(peer_ptrs)
    outs = (ctypes.c_void_p * world)(*[ctypes.c_void_p(int(x)) for x in peer_ptrs])
    with _on_device(dev):
        res = _lib.lib().aici_mha_varlen_fwd_peers(
            outs, ctypes.c_int(world), ctypes.c_int(head0), _p(q), _p(k), _p(v), _p(seqlens_q), _p(seqlens_k),
            ctypes.c_int(batch), ctypes.c_int(total_q), ctypes.c_int(k.shape[0]), ctypes.c_int(num_heads),
            ctypes.c_int(k.shape[1]), ctypes.c_int(head_size), ctypes.c_int(int(max_seqlen_q)),
            ctypes.c_int(int(max_seqlen_k)), ctypes.c_int64(q.stride(0)), ctypes.c_int64(q.stride(1)),
            ctypes.c_int64(k.stride(0)), ctypes.c_int64(k.stride(1)), ctypes.c_int64(v.stride(0)),
            ctypes.c_int64(v.stride(1)), ctypes.c_int64(total_heads * head_size), ctypes.c_int64(head_size),
            ctypes.c_float(softmax_scale), ctypes.c_int(1 if causal else 0), ctypes.c_int(_dtype(fn, q)),
            _stream(dev))
    _lib.check(fn, res)
