"""The native step-metadata builder (aici_batch_info_build, host code only: no GPU needed) against
the Python restatement of BatchInfoBuilder::finish (oracle/batch_info_ref.py)."""
import random

import pytest
import torch

from aici_b200 import batch_info
from aici_b200._lib import AiciError
from oracle import batch_info_ref

BS = 16


def make_entries(seed, n, pool_blocks=4096, max_len=300, single_frac=0.5):
    """Sequences as rLLM's allocator lays them out (paged/blocks.rs:122-127): each takes whole
    blocks from a shuffled pool; slot = block * 16 + offset."""
    rng = random.Random(seed)
    free = list(range(pool_blocks))
    rng.shuffle(free)
    entries = []
    for i in range(n):
        k_len = rng.randint(1, max_len)
        q_len = 1 if rng.random() < single_frac else rng.randint(1, k_len)
        blocks = [free.pop() for _ in range((k_len + BS - 1) // BS)]
        slots = [blocks[t // BS] * BS + t % BS for t in range(k_len)]
        query = [(k_len - q_len + j, rng.randint(0, 31999)) for j in range(q_len)]
        entries.append((1000 + i, query, slots))
    return entries


def build(entries, **kw):
    b = batch_info.BatchInfoBuilder(block_size=BS, max_model_len=kw.pop("max_model_len", 4096), **kw)
    for seq_id, query, slots in entries:
        b.add_entry(seq_id, query, slots)
    return b.finish(step_no=3)


def check_against_ref(bi, ref):
    assert bi.tokens.tolist() == ref["tokens"]
    assert bi.positions.tolist() == ref["positions"]
    assert bi.slot_mapping.tolist() == ref["slot_mapping"]
    assert bi.logit_idxs.tolist() == ref["logit_idxs"]
    assert bi.seqlens_q.tolist() == ref["seqlens_q"]
    assert bi.seqlens_k.tolist() == ref["seqlens_k"]
    assert bi.max_seqlen_q == ref["max_seqlen_q"] and bi.max_seqlen_k == ref["max_seqlen_k"]
    assert bi.paged_block_tables.tolist() == ref["paged_block_tables"]
    assert bi.paged_context_lens.tolist() == ref["paged_context_lens"]
    assert bi.paged_max_context_len == ref["paged_max_context_len"]
    assert bi.seqlen_multi == ref["seqlen_multi"] and bi.q_multi == ref["q_multi"]
    assert bi.seq_id_to_idx == ref["seq_id_to_idx"]


def test_hand_worked_step():
    """Two decode sequences around one 3-token prompt; expected values worked out by hand from
    batch_info.rs:196-315."""
    entries = [
        (7, [(35, 100)], list(range(160, 176)) + list(range(32, 48)) + [64, 65, 66, 67]),
        (8, [(0, 1), (1, 2), (2, 3)], [16, 17, 18]),
        (9, [(16, 5)], list(range(480, 496)) + [0]),
    ]
    bi = build(entries)
    assert bi.tokens.tolist() == [1, 2, 3, 100, 5]           # prompt first, decodes behind it
    assert bi.positions.tolist() == [0, 1, 2, 35, 16]
    assert bi.slot_mapping.tolist() == [16, 17, 18, 67, 0]
    assert bi.logit_idxs.tolist() == [2, 3, 4]
    assert bi.seqlens_q.tolist() == [0, 3] and bi.seqlens_k.tolist() == [0, 3]
    assert bi.gather_mapping.tolist() == [16, 17, 18]
    assert bi.paged_block_tables.tolist() == [[10, 2, 4], [30, 0, 0]]
    assert bi.paged_context_lens.tolist() == [36, 17]
    assert (bi.seqlen_multi, bi.q_multi, bi.paged_max_context_len) == (1, 3, 36)
    assert bi.seq_id_to_idx == {8: 0, 7: 1, 9: 2}
    assert bi.step_no == 3


@pytest.mark.parametrize("seed,n,single_frac", [(1, 1, 1.0), (2, 1, 0.0), (3, 17, 0.5), (4, 64, 0.9),
                                                (5, 40, 0.0), (6, 40, 1.0), (7, 200, 0.7)])
@pytest.mark.parametrize("paged_v", [1, 0])
def test_matches_reference_builder(seed, n, single_frac, paged_v):
    entries = make_entries(seed, n, single_frac=single_frac)
    bi = build(entries, paged_attn_kernel_v=paged_v)
    ref = batch_info_ref.finish(entries, BS, 4096, paged_attn_kernel_v=paged_v)
    check_against_ref(bi, ref)
    assert bi.gather_mapping.tolist() == ref["gather_mapping"]


def test_sections_are_aligned_and_disjoint():
    bi = build(make_entries(11, 33))
    lay = bi.layout
    offs = [lay.tokens_off, lay.positions_off, lay.slot_mapping_off, lay.logit_idxs_off,
            lay.seqlens_q_off, lay.seqlens_k_off, lay.gather_mapping_off, lay.block_tables_off,
            lay.context_lens_off, lay.total_bytes]
    assert all(o % 256 == 0 for o in offs)
    assert offs == sorted(offs)
    sizes = [lay.num_tokens * 4, lay.num_tokens * 8, lay.num_tokens * 4, lay.num_entries * 4,
             (lay.num_multitoken + 1) * 4, (lay.num_multitoken + 1) * 4, lay.gather_len * 4,
             lay.table_rows * lay.max_blocks_per_seq * 4, lay.table_rows * 4]
    for o, nxt, size in zip(offs, offs[1:], sizes):
        assert o + size <= nxt


def test_tables_for_all_and_no_gather_map():
    entries = make_entries(21, 30, single_frac=0.4)
    bi = build(entries, tables_for_all=True, gather_mapping=False)
    ref = batch_info_ref.finish(entries, BS, 4096)
    assert bi.gather_mapping.numel() == 0
    width = bi.layout.max_blocks_per_seq
    # decode rows: same blocks as the reference's, padded to the common width
    want = ref["paged_block_tables"]
    got = bi.paged_block_tables.tolist()
    for g, w, ctx in zip(got, want, ref["paged_context_lens"]):
        nb = (ctx + BS - 1) // BS
        assert g[:nb] == w[:nb] and all(v == 0 for v in g[nb:]) and len(g) == width
    assert bi.paged_context_lens.tolist() == ref["paged_context_lens"]
    # prefill rows: block of every 16th slot of the multi-token entries, in batch order
    by_id = {e[0]: e for e in entries}
    idx_to_id = {i: s for s, i in bi.seq_id_to_idx.items()}
    assert bi.multi_block_tables.shape[0] == bi.seqlen_multi
    for row in range(bi.seqlen_multi):
        slots = by_id[idx_to_id[row]][2]
        nb = (len(slots) + BS - 1) // BS
        assert bi.multi_block_tables[row, :nb].tolist() == [slots[t] // BS for t in range(0, len(slots), BS)]
        assert bi.multi_context_lens[row].item() == len(slots)


def test_default_positions_are_the_last_q_len():
    slots = torch.arange(64, 64 + 40, dtype=torch.int64)
    b = batch_info.BatchInfoBuilder(block_size=BS, max_model_len=4096)
    b.add_arrays(5, torch.tensor([11, 12, 13], dtype=torch.int32), slots)
    bi = b.finish()
    assert bi.positions.tolist() == [37, 38, 39]
    assert bi.slot_mapping.tolist() == [64 + 37, 64 + 38, 64 + 39]


def test_staging_buffers_are_reused_between_steps():
    b = batch_info.BatchInfoBuilder(block_size=BS, max_model_len=4096)
    outs = []
    for step in range(5):
        entries = make_entries(100 + step, 20)
        for e in entries:
            b.add_entry(*e)
        outs.append((b.finish(step), batch_info_ref.finish(entries, BS, 4096)))
    for bi, ref in outs:  # earlier results are not disturbed by later steps
        check_against_ref(bi, ref)


def test_errors_mirror_the_reference_asserts():
    b = batch_info.BatchInfoBuilder(block_size=BS, max_model_len=4096)
    with pytest.raises(AiciError, match="at least one sequence"):
        b.finish()
    with pytest.raises(AiciError, match="max_model_len"):
        build([(1, [(4096, 3)], [0])])
    with pytest.raises(AiciError, match="does not start a block"):
        build([(1, [(16, 3)], list(range(3, 19)) + [32])])  # first slot is not a block start
    with pytest.raises(AiciError, match="q_len <= k_len"):
        build([(1, [(0, 3), (1, 4)], [0])])
