"""KV-head sharding of the attention path over the GPUs of one box, and the one exchange it
needs: the gather of head outputs.

The reference has no multi-GPU code, only the hook that sizes the cache by kv heads per rank
(`get_num_heads_parallel = num_key_value_heads / tensor_parallel_size`,
rllm/rllm-cuda/src/llm/config.rs:49-51, with the divisibility check at :30-36).  Following that
hook, rank r of G owns kv heads [r*Hkv/G, (r+1)*Hkv/G) and the matching Hq/G query heads.  Cache
writes, block copies, decode and prefill then need no communication at all (block tables, slots
and cu_seqlens are the same on every rank); afterwards every rank needs all heads of the
attention output, which is one all-gather.

torch.distributed is the plumbing (backend "nccl" on GPUs; "gloo" in the CPU tests).  The
peer-mapped buffers of the fused gather come from the library's own C ABI (CUDA virtual-memory
allocations shared by file descriptor, CUDA IPC where that is unavailable), not from torch: a host
without libtorch maps them with the same four calls.
"""
import ctypes
from typing import List, Optional

import torch
import torch.distributed as dist

from dataclasses import dataclass


class ShardingError(RuntimeError):
    pass


@dataclass
class Shard:
    """KV-head sharding: rank r of `world` owns kv heads [r*Hkv/world, (r+1)*Hkv/world) and the
    matching query heads (the reference's get_num_heads_parallel, rllm-cuda/src/llm/config.rs:49-51)."""
    rank: int = 0
    world: int = 1

    def kv_slice(self, num_kv_heads: int) -> slice:
        if num_kv_heads % self.world != 0:
            raise ShardingError("num_kv_heads must divide by the world size")
        n = num_kv_heads // self.world
        return slice(self.rank * n, (self.rank + 1) * n)

    def q_slice(self, num_heads: int) -> slice:
        n = num_heads // self.world
        return slice(self.rank * n, (self.rank + 1) * n)


def check_world(num_heads: int, num_kv_heads: int, world: int) -> None:
    """Host-side validation before anything is launched (the reference's verify_args)."""
    if world < 1:
        raise ShardingError("world size must be positive")
    if num_kv_heads % world != 0:
        raise ShardingError("num_key_value_heads (%d) must be divisible by the world size (%d)"
                            % (num_kv_heads, world))
    if num_heads % num_kv_heads != 0:
        raise ShardingError("num_heads must be a multiple of num_kv_heads")


def current_shard(num_heads: int, num_kv_heads: int, group=None) -> Shard:
    if not dist.is_available() or not dist.is_initialized():
        return Shard(0, 1)
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    check_world(num_heads, num_kv_heads, world)
    return Shard(rank, world)


def shard_heads(t: torch.Tensor, shard: Shard, head_dim: int = 1) -> torch.Tensor:
    """This rank's contiguous slice of a [.., heads, ..] tensor along head_dim."""
    n = t.shape[head_dim]
    if n % shard.world != 0:
        raise ShardingError("%d heads do not divide over %d ranks" % (n, shard.world))
    per = n // shard.world
    return t.narrow(head_dim, shard.rank * per, per).contiguous()


def gather_heads(out_local: torch.Tensor, group=None, buffer: Optional[torch.Tensor] = None,
                 interleave: bool = True) -> torch.Tensor:
    """All-gather of per-rank head outputs [tokens, Hq/G, D].

    interleave=True returns [tokens, Hq, D] with heads in global order (one permuting copy after
    the collective); interleave=False returns the collective's own layout [G, tokens, Hq/G, D],
    which a row-parallel output projection can consume block by block without the copy."""
    if not dist.is_available() or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return out_local if interleave else out_local.unsqueeze(0)
    world = dist.get_world_size(group)
    tokens, h_local, d = out_local.shape
    if buffer is None:
        buffer = torch.empty(world, tokens, h_local, d, dtype=out_local.dtype, device=out_local.device)
    elif tuple(buffer.shape) != (world, tokens, h_local, d):
        raise ShardingError("gather buffer has the wrong shape")
    dist.all_gather_into_tensor(buffer.view(world * tokens, h_local, d), out_local.contiguous(), group=group)
    if not interleave:
        return buffer
    return buffer.permute(1, 0, 2, 3).reshape(tokens, world * h_local, d)


def exchange_bytes(payload: bytes, group=None) -> List[bytes]:
    """Every rank contributes `payload`; returns all ranks' payloads in rank order.  The channel is
    the process group's object all-gather (any channel would do: the C ABI only needs the 64 handle
    bytes to reach the other processes).  A rank that never joins makes the collective run into the
    group's timeout; that, and any other failure, surfaces as ShardingError instead of a hang."""
    if not dist.is_available() or not dist.is_initialized():
        raise ShardingError("exchange_bytes needs an initialised process group")
    world = dist.get_world_size(group)
    out: List[Optional[bytes]] = [None] * world
    try:
        dist.all_gather_object(out, bytes(payload), group=group)
    except Exception as e:  # noqa: BLE001 - timeouts and transport errors differ by backend
        raise ShardingError("handle exchange failed (is every rank alive?): %s: %s"
                            % (type(e).__name__, str(e)[:200])) from e
    if any(not isinstance(x, (bytes, bytearray)) or len(x) != len(payload) for x in out):
        raise ShardingError("handle exchange returned malformed entries")
    return [bytes(x) for x in out]


HANDLE_BYTES = 128  # AICI_PEER_HANDLE_BYTES


class _DevicePointer:
    """Lets torch view raw device memory (CUDA array interface, int16 elements)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes // 2,), "typestr": "<i2", "data": (int(ptr), False),
                                         "version": 2}


class PeerMemory:
    """`nbytes` of zero-filled device memory on every rank of `group`, each rank's block mapped into
    every other rank's process through the library's own calls (aici_peer_alloc / aici_peer_open:
    CUDA IPC handles, exchanged with `exchange_bytes`).  ptrs[r] is rank r's block as THIS process
    addresses it.  Set-up and tear-down only; never inside a step."""

    def __init__(self, nbytes: int, device, group=None):
        from . import _lib
        if not dist.is_initialized():
            raise ShardingError("PeerMemory needs an initialised process group")
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.device = torch.device(device)
        self.nbytes = int(nbytes)
        self._lib = _lib
        self._own = ctypes.c_void_p(0)
        self._opened: List[int] = []
        self.ptrs: List[int] = []
        handle = (ctypes.c_ubyte * HANDLE_BYTES)()
        err: Optional[str] = None
        with torch.cuda.device(self.device):
            try:
                _lib.check("aici_peer_alloc", _lib.lib().aici_peer_alloc(
                    ctypes.c_size_t(self.nbytes), ctypes.byref(self._own), handle))
            except _lib.AiciError as e:
                err = str(e)
            # bytes 4..7 of a handle say how the block is shared (1: virtual-memory allocation through
            # a duplicated file descriptor, 2: CUDA IPC handle of a cudaMalloc block)
            self.kind = int.from_bytes(bytes(handle)[4:8], "little") if err is None else 0
            # every rank takes part in the exchange even if its own allocation failed, so that
            # nobody waits for a rank that has already given up
            handles = exchange_bytes(bytes(handle) if err is None else b"\0" * HANDLE_BYTES, self.group)
            if err is None and any(h == b"\0" * HANDLE_BYTES for h in handles):
                err = "another rank could not allocate its peer buffer"
            if err is None:
                for r, h in enumerate(handles):
                    if r == self.rank:
                        self.ptrs.append(int(self._own.value))
                        continue
                    out = ctypes.c_void_p(0)
                    try:
                        _lib.check("aici_peer_open", _lib.lib().aici_peer_open(
                            (ctypes.c_ubyte * HANDLE_BYTES).from_buffer_copy(h), ctypes.byref(out)))
                    except _lib.AiciError as e:
                        err = str(e)
                        break
                    self._opened.append(int(out.value))
                    self.ptrs.append(int(out.value))
            # agree on the outcome: one failed mapping anywhere means nobody uses the buffers
            oks = exchange_bytes(b"\1" if err is None else b"\0", self.group)
            if any(o != b"\1" for o in oks):
                self.close(meet=False)
                raise ShardingError(err or "another rank could not map the peer buffers")

    def view(self, offset: int, shape, dtype=torch.bfloat16, rank: Optional[int] = None) -> torch.Tensor:
        """A tensor over this rank's own block (or, with `rank`, over that rank's block as mapped here)."""
        n = 1
        for d in shape:
            n *= int(d)
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        if offset % 16 or offset + nbytes > self.nbytes:
            raise ShardingError("view outside the peer block")
        base = self.ptrs[self.rank if rank is None else rank] + offset
        t = torch.as_tensor(_DevicePointer(base, nbytes), device=self.device)
        return t.view(dtype).view(*shape)

    def close(self, meet: bool = True) -> None:
        """Unmaps the peers' blocks, meets the other ranks, frees the own block (in that order: a
        block must not be freed while a peer still has it mapped)."""
        lib = self._lib.lib()

        def quietly(name, res):  # tear-down goes on past an error, but the message must not leak
            try:
                self._lib.check(name, res)
            except self._lib.AiciError:
                pass
        with torch.cuda.device(self.device):
            torch.cuda.synchronize(self.device)
            for p in self._opened:
                quietly("aici_peer_close", lib.aici_peer_close(ctypes.c_void_p(p)))
            self._opened = []
            if meet and dist.is_initialized():
                try:
                    dist.barrier(group=self.group)
                except Exception:  # noqa: BLE001 - a dead peer must not keep this rank from freeing
                    pass
            if self._own.value:
                quietly("aici_peer_free", lib.aici_peer_free(self._own))
                self._own = ctypes.c_void_p(0)
        self.ptrs = []


class PeerGather:
    """Output buffers [rows, total_heads, head_size] on every rank of `group`, mapped into every
    peer's address space (PeerMemory), plus the flag array of the library's barrier.  The attention
    entry points `*_peers` store each rank's heads straight into all ranks' buffers; `barrier()`
    (bounded wait on the device) is the only synchronisation before `tensor` holds all heads.

    There are `buffers` output buffers (default 2) used in turn: a peer may start its next step
    while this rank still reads the current one, so consecutive steps write different buffers.
    `flip()` moves on to the next buffer; with two buffers and one barrier per step, a buffer is
    written again only after every rank has passed the barrier of the step in between, i.e. after
    its readers (stream-ordered before that step's kernels) are done."""

    FLAG_BYTES = 256

    def __init__(self, rows: int, total_heads: int, head_size: int, device, group=None,
                 dtype=torch.bfloat16, buffers: int = 2):
        if not dist.is_initialized():
            raise ShardingError("PeerGather needs an initialised process group")
        grp = group if group is not None else dist.group.WORLD
        world = dist.get_world_size(grp)
        if total_heads % world != 0:
            raise ShardingError("%d heads do not divide over %d ranks" % (total_heads, world))
        if buffers < 1:
            raise ShardingError("at least one buffer is needed")
        self.total_heads = total_heads
        self.heads_per_rank = total_heads // world
        self.shape = (rows, total_heads, head_size)
        elem = torch.empty((), dtype=dtype).element_size()
        self._buf_bytes = (rows * total_heads * head_size * elem + 255) // 256 * 256
        self.mem = PeerMemory(self.FLAG_BYTES + buffers * self._buf_bytes, device, grp)
        self.group, self.world, self.rank = self.mem.group, self.mem.world, self.mem.rank
        self.buffers = buffers
        self.tensors = [self.mem.view(self.FLAG_BYTES + i * self._buf_bytes, self.shape, dtype)
                        for i in range(buffers)]
        self._ptrs = [[p + self.FLAG_BYTES + i * self._buf_bytes for p in self.mem.ptrs] for i in range(buffers)]
        self.flag_ptrs = list(self.mem.ptrs)  # the first 32 words of each block, zero after allocation
        self.cur = 0

    @property
    def tensor(self) -> torch.Tensor:
        return self.tensors[self.cur]

    @property
    def ptrs(self) -> List[int]:
        return self._ptrs[self.cur]

    def flip(self) -> None:
        self.cur = (self.cur + 1) % self.buffers

    @property
    def head0(self) -> int:
        return self.rank * self.heads_per_rank

    def flag_array(self):
        return (ctypes.c_void_p * self.world)(*[ctypes.c_void_p(x) for x in self.flag_ptrs])

    def barrier(self) -> None:
        """Enqueue the cross-rank barrier on the current stream (bounded wait on the device)."""
        from . import _lib
        dev = self.mem.device
        with torch.cuda.device(dev):
            res = _lib.lib().aici_peer_barrier(self.flag_array(), ctypes.c_int(self.world), ctypes.c_int(self.rank),
                                               ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
        _lib.check("peer_barrier", res)

    def close(self) -> None:
        self.tensors = []
        self.mem.close()
