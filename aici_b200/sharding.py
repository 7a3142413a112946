"""KV-head sharding of the attention path over the GPUs of one box, and the one exchange it
needs: the gather of head outputs.

The reference has no multi-GPU code, only the hook that sizes the cache by kv heads per rank
(`get_num_heads_parallel = num_key_value_heads / tensor_parallel_size`,
rllm/rllm-cuda/src/llm/config.rs:49-51, with the divisibility check at :30-36).  Following that
hook, rank r of G owns kv heads [r*Hkv/G, (r+1)*Hkv/G) and the matching Hq/G query heads.  Cache
writes, block copies, decode and prefill then need no communication at all (block tables, slots
and cu_seqlens are the same on every rank); afterwards every rank needs all heads of the
attention output, which is one all-gather.

torch.distributed is the plumbing (backend "nccl" on GPUs; "gloo" in the CPU tests).
"""
from typing import Optional

import torch
import torch.distributed as dist

from .workloads import Shard


class ShardingError(RuntimeError):
    pass


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


class PeerGather:
    """Output buffer [rows, total_heads, head_size] allocated in symmetric memory on every rank of
    `group` and mapped into every peer's address space (torch.distributed symmetric memory over
    NVLink).  The attention entry points `*_peers` store each rank's heads straight into all of
    these buffers; `barrier()` (a signal exchange on the current stream, with a timeout) is the only
    synchronisation before `tensor` holds all heads on every rank."""

    def __init__(self, rows: int, total_heads: int, head_size: int, device, group=None,
                 dtype=torch.bfloat16):
        import torch.distributed._symmetric_memory as symm_mem
        if not dist.is_initialized():
            raise ShardingError("PeerGather needs an initialised process group")
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        if total_heads % self.world != 0:
            raise ShardingError("%d heads do not divide over %d ranks" % (total_heads, self.world))
        self.total_heads = total_heads
        self.heads_per_rank = total_heads // self.world
        self.tensor = symm_mem.empty((rows, total_heads, head_size), dtype=dtype, device=device)
        self.handle = symm_mem.rendezvous(self.tensor, self.group)
        self.ptrs = [int(x) for x in self.handle.buffer_ptrs]
        if len(self.ptrs) != self.world or self.ptrs[self.rank] != self.tensor.data_ptr():
            raise ShardingError("symmetric memory rendezvous returned unexpected buffer pointers")
        # flags of the library's own barrier kernel: 16 slots per rank, zero, peer-mapped
        self._flags = symm_mem.empty((16,), dtype=torch.int32, device=device)
        self._flags.zero_()
        self._flag_handle = symm_mem.rendezvous(self._flags, self.group)
        self._flag_ptrs = [int(x) for x in self._flag_handle.buffer_ptrs]
        torch.cuda.synchronize(device)
        self.handle.barrier(channel=0, timeout_ms=60000)  # every rank's flags are zero before first use

    @property
    def head0(self) -> int:
        return self.rank * self.heads_per_rank

    def barrier(self) -> None:
        """Enqueue the cross-rank barrier on the current stream (bounded wait on the device)."""
        import ctypes
        from . import _lib
        arr = (ctypes.c_void_p * self.world)(*[ctypes.c_void_p(x) for x in self._flag_ptrs])
        dev = self.tensor.device
        with torch.cuda.device(dev):
            res = _lib.lib().aici_peer_barrier(arr, ctypes.c_int(self.world), ctypes.c_int(self.rank),
                                               ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
        _lib.check("peer_barrier", res)
