"""Pure-Python restatement of rLLM's step-metadata builder -- TEST INFRASTRUCTURE ONLY.

Follows BatchInfoBuilder::finish (rllm-cuda/src/llm/paged/batch_info.rs:196-315), to_offsets
(rllm-cuda/src/llm/kernels.rs:10-21) and pad_to_multiple (rllm-base/src/util.rs:113-123) with
plain lists, the way the reference builds its Vecs before uploading them.  Entries are
(seq_id, [(position, token), ...], [kv_slot, ...]) triples, i.e. BatchEntry (:93-97).
Parity is unpinned by stored vectors (the reference has no test for this function); the checks
are the structural properties its consumers rely on plus hand-worked cases in the tests.
"""


def to_offsets(lengths):
    """kernels.rs:10-21: (max length, exclusive prefix sums with the total appended)."""
    offsets, total, longest = [], 0, 0
    for n in lengths:
        longest = max(longest, n)
        offsets.append(total)
        total += n
    offsets.append(total)
    return longest, offsets


def pad_to_multiple(row, multiple):
    """util.rs:113-123 (zero fill).  A multiple of 0 cannot occur for a non-empty row."""
    rem = len(row) % multiple if multiple else 0
    return row + [0] * (multiple - rem) if rem else row


def finish(entries, block_size, max_model_len, paged_attn_kernel_v=1):
    assert len(entries) > 0
    if paged_attn_kernel_v > 0:  # :209-221, single-token entries move to the back, order kept
        multi = [e for e in entries if len(e[1]) != 1]
        single = [e for e in entries if len(e[1]) == 1]
        entries = multi + single
        num_multitoken = len(multi)
    else:
        entries = list(entries)
        num_multitoken = len(entries)

    out = dict(positions=[], tokens=[], logit_idxs=[], gather_mapping=[], slot_mapping=[],
               seq_id_to_idx={})
    lens_q, lens_k, tables, context_lens = [], [], [], []
    first_single_token = 0
    for idx, (seq_id, query, kv_slots) in enumerate(entries):
        out["seq_id_to_idx"][seq_id] = idx
        off = len(kv_slots) - len(query)
        for qidx, (tpos, token) in enumerate(query):
            assert tpos < max_model_len
            out["positions"].append(tpos)
            out["tokens"].append(token)
            out["slot_mapping"].append(kv_slots[off + qidx])
        out["logit_idxs"].append(len(out["tokens"]) - 1)
        if idx < num_multitoken:  # :239-245
            out["gather_mapping"] += list(kv_slots)
            first_single_token = len(out["tokens"])
            lens_q.append(len(query))
            lens_k.append(len(kv_slots))
        else:  # :246-262
            context_lens.append(len(kv_slots))
            row = []
            for t in range(0, len(kv_slots), block_size):
                assert kv_slots[t] % block_size == 0
                row.append(kv_slots[t] // block_size)
            tables.append(row)
    out["max_seqlen_q"], out["seqlens_q"] = to_offsets(lens_q)
    out["max_seqlen_k"], out["seqlens_k"] = to_offsets(lens_k)
    width = max((len(r) for r in tables), default=0)
    out["paged_block_tables"] = [pad_to_multiple(r, width) for r in tables]
    out["paged_context_lens"] = context_lens
    out["paged_max_context_len"] = max(context_lens, default=0)
    out["seqlen_multi"] = num_multitoken
    out["q_multi"] = first_single_token
    return out
