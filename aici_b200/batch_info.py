"""Host-side mirror of rLLM's BatchInfoBuilder / BatchInfo for the attention path.

Same roles and field names as rllm-cuda/src/llm/paged/batch_info.rs (BatchEntry :93-97,
BatchInfoBuilder :88-315, BatchInfo :18-43).  The work is done by the native builder behind
`aici_batch_info_build` (include/aici_b200.h): every index tensor of the step is written into one
page-locked staging buffer and reaches the device with one copy; the fields of the returned
`BatchInfo` are views into that one device buffer.
"""
import ctypes
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from . import _lib
from ._lib import AiciError

PAGED_DECODE = 1
TABLES_FOR_ALL = 2
NO_GATHER_MAP = 4


class _Entry(ctypes.Structure):
    _fields_ = [("seq_id", ctypes.c_int64), ("tokens", ctypes.c_void_p),
                ("positions", ctypes.c_void_p), ("kv_slots", ctypes.c_void_p),
                ("q_len", ctypes.c_int32), ("k_len", ctypes.c_int32)]


class Layout(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int64) for n in (
        "total_bytes", "tokens_off", "positions_off", "slot_mapping_off", "logit_idxs_off",
        "seqlens_q_off", "seqlens_k_off", "gather_mapping_off", "block_tables_off",
        "context_lens_off")] + [(n, ctypes.c_int32) for n in (
            "num_entries", "num_tokens", "num_multitoken", "q_multi", "max_seqlen_q", "max_seqlen_k",
            "gather_len", "num_paged", "table_rows", "paged_row0", "max_blocks_per_seq",
            "paged_max_context_len")]


class BatchInfo:
    """Index tensors of one step (batch_info.rs:18-43); all views of `buffer`."""

    def __init__(self, buffer: torch.Tensor, lay: Layout, order: List[int], seq_ids: List[int],
                 block_size: int, step_no: int):
        def sec(off, count, dtype):
            nbytes = count * torch.empty((), dtype=dtype).element_size()
            return buffer[off:off + nbytes].view(dtype)

        self.buffer = buffer
        self.layout = lay
        self.step_no = step_no
        self.tokens = sec(lay.tokens_off, lay.num_tokens, torch.int32)
        self.positions = sec(lay.positions_off, lay.num_tokens, torch.int64)
        self.slot_mapping = sec(lay.slot_mapping_off, lay.num_tokens, torch.int32)
        self.logit_idxs = sec(lay.logit_idxs_off, lay.num_entries, torch.int32)
        self.seqlens_q = sec(lay.seqlens_q_off, lay.num_multitoken + 1, torch.int32)
        self.seqlens_k = sec(lay.seqlens_k_off, lay.num_multitoken + 1, torch.int32)
        self.gather_mapping = sec(lay.gather_mapping_off, lay.gather_len, torch.int32)
        tables = sec(lay.block_tables_off, lay.table_rows * lay.max_blocks_per_seq, torch.int32)
        tables = tables.view(lay.table_rows, lay.max_blocks_per_seq)
        lens = sec(lay.context_lens_off, lay.table_rows, torch.int32)
        # rows of the single-token entries, as the reference's fields of the same name
        self.paged_block_tables = tables[lay.paged_row0:]
        self.paged_context_lens = lens[lay.paged_row0:]
        # rows of the multi-token entries (empty unless TABLES_FOR_ALL was asked for)
        self.multi_block_tables = tables[:lay.paged_row0]
        self.multi_context_lens = lens[:lay.paged_row0]
        self.paged_block_size = block_size
        self.paged_max_context_len = lay.paged_max_context_len
        self.max_seqlen_q = lay.max_seqlen_q
        self.max_seqlen_k = lay.max_seqlen_k
        self.seqlen_multi = lay.num_multitoken
        self.q_multi = lay.q_multi
        self.entry_order = order
        self.seq_id_to_idx: Dict[int, int] = {seq_ids[e]: i for i, e in enumerate(order)}


class BatchInfoBuilder:
    """Collects the running sequences of a step, then `finish()` lays them out and uploads them.

    `paged_attn_kernel_v`, `block_size`, `max_model_len` are the config fields the reference
    reads (batch_info.rs:209, 223, 249).  The staging buffers (host, page-locked when a device
    is given) are kept and grown between steps, so a steady-state step allocates nothing.
    """

    def __init__(self, block_size: int = 16, max_model_len: int = 1 << 20,
                 paged_attn_kernel_v: int = 1, device: Optional[torch.device] = None,
                 tables_for_all: bool = False, gather_mapping: bool = True):
        self.block_size = block_size
        self.max_model_len = max_model_len
        self.flags = ((PAGED_DECODE if paged_attn_kernel_v > 0 else 0) |
                      (TABLES_FOR_ALL if tables_for_all else 0) |
                      (0 if gather_mapping else NO_GATHER_MAP))
        self.device = device
        self.entries: List[Tuple[int, torch.Tensor, Optional[torch.Tensor], torch.Tensor]] = []
        # two staging buffers used in turn; each remembers the event of its last upload
        self._staging: List[Optional[torch.Tensor]] = [None, None]
        self._uploaded: List[Optional[torch.cuda.Event]] = [None, None]
        self._turn = 0

    def add_entry(self, seq_id: int, query_pos_token: Sequence[Tuple[int, int]],
                  kv_slots: Sequence[int]) -> "BatchInfoBuilder":
        """One BatchEntry (batch_info.rs:93-97): (position, token) pairs of this step's query
        tokens and the cache slot of every token of the sequence."""
        pos = torch.tensor([p for p, _ in query_pos_token], dtype=torch.int64)
        tok = torch.tensor([t for _, t in query_pos_token], dtype=torch.int32)
        slots = torch.as_tensor(kv_slots, dtype=torch.int64).contiguous()
        self.entries.append((int(seq_id), tok, pos, slots))
        return self

    def add_arrays(self, seq_id: int, tokens: torch.Tensor, kv_slots: torch.Tensor,
                   positions: Optional[torch.Tensor] = None) -> "BatchInfoBuilder":
        """Same entry from ready-made CPU arrays (int32 tokens, int64 slots); positions default to
        the last len(tokens) positions of the sequence, which is what sched_out produces
        (batch_info.rs:121-140)."""
        self.entries.append((int(seq_id), tokens.to(torch.int32).contiguous(),
                             None if positions is None else positions.to(torch.int64).contiguous(),
                             kv_slots.to(torch.int64).contiguous()))
        return self

    def _c_entries(self):
        arr = (_Entry * max(len(self.entries), 1))()
        for i, (seq_id, tok, pos, slots) in enumerate(self.entries):
            arr[i].seq_id = seq_id
            arr[i].tokens = tok.data_ptr()
            arr[i].positions = 0 if pos is None else pos.data_ptr()
            arr[i].kv_slots = slots.data_ptr()
            arr[i].q_len = tok.numel()
            arr[i].k_len = slots.numel()
        return arr

    def finish(self, step_no: int = 0) -> BatchInfo:
        """BatchInfoBuilder::finish (batch_info.rs:196-315).  Clears the entry list."""
        fn = "BatchInfoBuilder.finish"
        n = len(self.entries)
        arr = self._c_entries()
        lay = Layout()
        lib = _lib.lib()
        _lib.check(fn, lib.aici_batch_info_layout(arr, ctypes.c_int(n), ctypes.c_int(self.flags),
                                                  ctypes.c_int(self.block_size),
                                                  ctypes.c_int64(self.max_model_len), ctypes.byref(lay)))
        need = max(int(lay.total_bytes), 256)
        on_gpu = self.device is not None and torch.device(self.device).type == "cuda"
        turn = self._turn
        self._turn ^= 1
        if self._staging[turn] is None or self._staging[turn].numel() < need:
            self._staging[turn] = torch.empty(max(need * 2, 1 << 16), dtype=torch.uint8,
                                              pin_memory=on_gpu)
        elif self._uploaded[turn] is not None:
            self._uploaded[turn].synchronize()  # the copy that last read this buffer is done
        staging = self._staging[turn]
        order = (ctypes.c_int32 * n)()
        if on_gpu:
            dev = torch.device(self.device)
            with torch.cuda.device(dev):
                buffer = torch.empty(need, dtype=torch.uint8, device=dev)
                _lib.check(fn, lib.aici_batch_info_build(
                    arr, ctypes.c_int(n), ctypes.c_int(self.flags), ctypes.c_int(self.block_size),
                    ctypes.c_int64(self.max_model_len), ctypes.c_void_p(staging.data_ptr()),
                    ctypes.c_size_t(staging.numel()), ctypes.c_void_p(buffer.data_ptr()),
                    ctypes.c_size_t(buffer.numel()), ctypes.byref(lay), order,
                    ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)))
                ev = torch.cuda.Event()
                ev.record()
                self._uploaded[turn] = ev
        else:
            _lib.check(fn, lib.aici_batch_info_build(
                arr, ctypes.c_int(n), ctypes.c_int(self.flags), ctypes.c_int(self.block_size),
                ctypes.c_int64(self.max_model_len), ctypes.c_void_p(staging.data_ptr()),
                ctypes.c_size_t(staging.numel()), ctypes.c_void_p(0), ctypes.c_size_t(0),
                ctypes.byref(lay), order, ctypes.c_void_p(0)))
            buffer = staging[:need].clone()
        seq_ids = [e[0] for e in self.entries]
        self.entries = []
        return BatchInfo(buffer, lay, list(order), seq_ids, self.block_size, step_no)
