"""Seeded synthetic inputs for the five attention-path configurations (benchmark and test harness;
not part of the product package).

The reference publishes no dataset for this path; these generators ARE the inputs: shapes,
context-length distributions and block-table construction follow the configuration list the
benchmark is quoted on.  Values are N(0,1) drawn in fp32 from a seeded torch.Generator on
the target device and cast to bf16.  Every rank of a multi-GPU run draws the same full
tensors and keeps its own KV heads (`shard`), so results are comparable element by element
across GPU counts.

Block tables are built the way rLLM builds them (rllm-cuda/src/llm/paged/batch_info.rs:244-291):
one row per sequence, zero-padded to the longest; slot = physical_block * block_size + offset
(paged/blocks.rs:122-127).
"""
import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch

from aici_b200.sharding import Shard

HEAD_DIM = 128
BLOCK_SIZE = 16
X = 8  # 16 bytes of bf16


def _gen(device, seed: int) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return g


def randn_bf16(shape, device, gen: torch.Generator, chunk: int = 1 << 26) -> torch.Tensor:
    """N(0,1) in fp32, cast to bf16, generated in chunks to bound the fp32 temporary."""
    n = 1
    for s in shape:
        n *= int(s)
    out = torch.empty(n, dtype=torch.bfloat16, device=device)
    for i in range(0, n, chunk):
        m = min(chunk, n - i)
        out[i:i + m] = torch.randn(m, dtype=torch.float32, device=device, generator=gen).to(torch.bfloat16)
    return out.view(*shape)


@dataclass
class DecodeWorkload:
    name: str
    query: torch.Tensor          # [S, Hq_local, D]
    key_cache: torch.Tensor      # [nblk, Hkv_local, D/8, 16, 8]
    value_cache: torch.Tensor    # [nblk, Hkv_local, D, 16]
    block_tables: torch.Tensor   # int32 [S, max_blocks]
    context_lens: torch.Tensor   # int32 [S]
    new_key: torch.Tensor        # [S, Hkv_local, D]  token written at position ctx-1
    new_value: torch.Tensor
    slot_mapping: torch.Tensor   # int32 [S]
    num_kv_heads: int
    num_heads: int
    scale: float
    max_context_len: int
    context_list: List[int] = field(default_factory=list)

    def algorithmic_bytes(self) -> int:
        """K and V once per (seq, kv head), q in, out, block table, context lens."""
        hkv, hq = self.num_kv_heads, self.num_heads
        kv = sum(self.context_list) * 2 * hkv * HEAD_DIM * 2
        qo = len(self.context_list) * hq * HEAD_DIM * 2 * 2
        bt = sum((c + BLOCK_SIZE - 1) // BLOCK_SIZE for c in self.context_list) * 4
        return kv + qo + bt + 4 * len(self.context_list)

    def cache_write_bytes(self) -> int:
        """reshape_and_cache of the new tokens: K and V, read + write."""
        return len(self.context_list) * self.num_kv_heads * HEAD_DIM * 2 * 2 * 2


def draw_context_lens(kind: str, n: int, lo: int, hi: int, seed: int) -> List[int]:
    g = torch.Generator()
    g.manual_seed(seed)
    if kind == "uniform":
        return torch.randint(lo, hi + 1, (n,), generator=g).tolist()
    if kind == "loguniform":
        u = torch.rand(n, generator=g, dtype=torch.float64)
        v = torch.exp(math.log(lo) + u * (math.log(hi) - math.log(lo))).round().to(torch.int64)
        return v.clamp_(lo, hi).tolist()
    raise ValueError(kind)


def build_block_tables(context_list: List[int], pool_blocks: int, seed: int,
                       first_block: int = 0) -> Tuple[torch.Tensor, List[List[int]]]:
    """Each sequence takes ceil(ctx/16) consecutive entries of one seeded permutation of the
    pool; rows are zero-padded to the longest."""
    g = torch.Generator()
    g.manual_seed(seed)
    perm = (torch.randperm(pool_blocks - first_block, generator=g) + first_block).tolist()
    rows, pos = [], 0
    for c in context_list:
        n = (c + BLOCK_SIZE - 1) // BLOCK_SIZE
        assert pos + n <= len(perm), "block pool too small for the drawn contexts"
        rows.append(perm[pos:pos + n])
        pos += n
    width = max((len(r) for r in rows), default=0)
    table = torch.zeros(len(rows), max(width, 1), dtype=torch.int32)
    for i, r in enumerate(rows):
        table[i, :len(r)] = torch.tensor(r, dtype=torch.int32)
    return table, rows


def make_decode(name: str, device, *, num_seqs: int, num_heads: int, num_kv_heads: int,
                ctx_kind: str, ctx_lo: int, ctx_hi: int, pool_blocks: int, seed: int,
                shard: Optional[Shard] = None) -> DecodeWorkload:
    shard = shard or Shard()
    ctx = draw_context_lens(ctx_kind, num_seqs, ctx_lo, ctx_hi, seed + 1)
    table, rows = build_block_tables(ctx, pool_blocks, seed + 2)
    g = _gen(device, seed + 3)
    kc = randn_bf16((pool_blocks, num_kv_heads, HEAD_DIM // X, BLOCK_SIZE, X), device, g)
    vc = randn_bf16((pool_blocks, num_kv_heads, HEAD_DIM, BLOCK_SIZE), device, g)
    q = randn_bf16((num_seqs, num_heads, HEAD_DIM), device, g)
    nk = randn_bf16((num_seqs, num_kv_heads, HEAD_DIM), device, g)
    nv = randn_bf16((num_seqs, num_kv_heads, HEAD_DIM), device, g)
    if shard.world > 1:
        ks, qs = shard.kv_slice(num_kv_heads), shard.q_slice(num_heads)
        kc, vc = kc[:, ks].contiguous(), vc[:, ks].contiguous()
        q, nk, nv = q[:, qs].contiguous(), nk[:, ks].contiguous(), nv[:, ks].contiguous()
    slots = [rows[i][(c - 1) // BLOCK_SIZE] * BLOCK_SIZE + (c - 1) % BLOCK_SIZE
             for i, c in enumerate(ctx)]
    return DecodeWorkload(
        name=name, query=q, key_cache=kc, value_cache=vc,
        block_tables=table.to(device), context_lens=torch.tensor(ctx, dtype=torch.int32, device=device),
        new_key=nk, new_value=nv, slot_mapping=torch.tensor(slots, dtype=torch.int32, device=device),
        num_kv_heads=kc.shape[1], num_heads=q.shape[1], scale=1.0 / math.sqrt(HEAD_DIM),
        max_context_len=max(ctx) if ctx else 0, context_list=ctx)


def decode_llama2_7b(device, shard: Optional[Shard] = None, num_seqs: int = 64,
                     pool_blocks: int = 16384) -> DecodeWorkload:
    """Config 2: batch 64, 32 heads MHA, contexts uniform in [512, 4096], 16384-block pool."""
    return make_decode("decode_llama2_7b_b64_mha32_ctx512-4096", device, num_seqs=num_seqs,
                       num_heads=32, num_kv_heads=32, ctx_kind="uniform", ctx_lo=512, ctx_hi=4096,
                       pool_blocks=pool_blocks, seed=2000, shard=shard)


def decode_llama3_8b(device, shard: Optional[Shard] = None, num_seqs: int = 256,
                     pool_blocks: int = 65536) -> DecodeWorkload:
    """Config 3: batch 256, 32 q / 8 kv heads, contexts log-uniform in [128, 8192]."""
    return make_decode("decode_llama3_8b_b256_gqa32-8_ctx128-8192", device, num_seqs=num_seqs,
                       num_heads=32, num_kv_heads=8, ctx_kind="loguniform", ctx_lo=128, ctx_hi=8192,
                       pool_blocks=pool_blocks, seed=3000, shard=shard)


def decode_mixed_step(device, shard: Optional[Shard] = None, num_seqs: int = 192,
                      pool_blocks: int = 131072) -> DecodeWorkload:
    """Decode part of config 5: 192 sequences, contexts uniform in [256, 16384], 32 q / 8 kv."""
    return make_decode("decode_mixed_b192_gqa32-8_ctx256-16384", device, num_seqs=num_seqs,
                       num_heads=32, num_kv_heads=8, ctx_kind="uniform", ctx_lo=256, ctx_hi=16384,
                       pool_blocks=pool_blocks, seed=5000, shard=shard)


@dataclass
class PrefillWorkload:
    name: str
    q: torch.Tensor             # [total_q, Hq_local, D]
    k: torch.Tensor             # [total_k, Hkv_local, D]
    v: torch.Tensor
    cu_seqlens_q: torch.Tensor  # int32 [b+1]
    cu_seqlens_k: torch.Tensor
    max_seqlen_q: int
    max_seqlen_k: int
    scale: float
    lens_q: List[int] = field(default_factory=list)
    lens_k: List[int] = field(default_factory=list)

    def flops(self) -> float:
        """4 * D * Hq * (number of visible (row, column) pairs); masked work not counted."""
        hq = self.q.shape[1]
        vis = 0
        for lq, lk in zip(self.lens_q, self.lens_k):
            # row r sees min(lk, r + 1 + lk - lq) columns, clipped at 0
            for_first = lk - lq  # columns before the diagonal band
            if for_first >= 0:
                vis += lq * for_first + lq * (lq + 1) // 2
            else:
                n = lk  # only the last lk rows see anything
                vis += n * (n + 1) // 2
        return 4.0 * HEAD_DIM * hq * vis


def make_prefill(name: str, device, *, lens_q: List[int], lens_k: List[int], num_heads: int,
                 num_kv_heads: int, seed: int, shard: Optional[Shard] = None) -> PrefillWorkload:
    shard = shard or Shard()
    g = _gen(device, seed)
    tq, tk = sum(lens_q), sum(lens_k)
    q = randn_bf16((tq, num_heads, HEAD_DIM), device, g)
    k = randn_bf16((tk, num_kv_heads, HEAD_DIM), device, g)
    v = randn_bf16((tk, num_kv_heads, HEAD_DIM), device, g)
    if shard.world > 1:
        ks, qs = shard.kv_slice(num_kv_heads), shard.q_slice(num_heads)
        q, k, v = q[:, qs].contiguous(), k[:, ks].contiguous(), v[:, ks].contiguous()

    def cu(lens):
        t = torch.zeros(len(lens) + 1, dtype=torch.int32)
        t[1:] = torch.tensor(lens, dtype=torch.int64).cumsum(0).to(torch.int32)
        return t.to(device)

    return PrefillWorkload(name=name, q=q, k=k, v=v, cu_seqlens_q=cu(lens_q), cu_seqlens_k=cu(lens_k),
                           max_seqlen_q=max(lens_q), max_seqlen_k=max(lens_k),
                           scale=1.0 / math.sqrt(HEAD_DIM), lens_q=list(lens_q), lens_k=list(lens_k))


def prefill_small(device, shard: Optional[Shard] = None) -> PrefillWorkload:
    """Config 1: 4 packed sequences of 64/128/256/512 tokens, 32 heads MHA."""
    lens = [64, 128, 256, 512]
    return make_prefill("prefill_4seq_64-512_mha32", device, lens_q=lens, lens_k=lens, num_heads=32,
                        num_kv_heads=32, seed=1000, shard=shard)


def prefill_long(device, shard: Optional[Shard] = None, seqlen: int = 32768) -> PrefillWorkload:
    """Config 4: 2 sequences of 32768 tokens, 64 q / 8 kv heads."""
    lens = [seqlen, seqlen]
    return make_prefill("prefill_2x%d_gqa64-8" % seqlen, device, lens_q=lens, lens_k=lens,
                        num_heads=64, num_kv_heads=8, seed=4000, shard=shard)


def prefill_mixed_chunks(device, shard: Optional[Shard] = None, cached: int = 0) -> PrefillWorkload:
    """Prefill part of config 5: 8 chunks of 512 query tokens, 32 q / 8 kv heads; `cached`
    extra key tokens per chunk already in the cache (k_len = cached + 512) exercise the
    bottom-right aligned mask."""
    return make_prefill("prefill_8x512_gqa32-8_cached%d" % cached, device, lens_q=[512] * 8,
                        lens_k=[512 + cached] * 8, num_heads=32, num_kv_heads=8, seed=5100, shard=shard)


def fork_block_mapping(rows: List[List[int]], n_parents: int, n_children: int, free_blocks: List[int],
                       whole_sequence: bool = False) -> Dict[int, List[int]]:
    """AICI fork: each of the first n_parents sequences forks n_children children.  rLLM
    copies only the shared LAST block per child on the next append
    (paged/blocks.rs:221-233); whole_sequence=True copies every block (bandwidth variant)."""
    mapping: Dict[int, List[int]] = {}
    it = iter(free_blocks)
    for r in rows[:n_parents]:
        srcs = r if whole_sequence else r[-1:]
        for s in srcs:
            mapping.setdefault(s, [])
            for _ in range(n_children):
                mapping[s].append(next(it))
    return mapping
