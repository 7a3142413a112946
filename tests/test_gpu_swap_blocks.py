"""GPU parity tests (bit-exact) for swap_blocks through the C ABI: device <-> page-locked host
(kernel over PCIe), device <-> pageable host (copy engine), device <-> device -- against the CPU
oracle and against the reference's own swap_blocks (kernels/vllm/cache_kernels.cu:12-50) run on the
same inputs through the comparator library."""
import ctypes
import os

import pytest
import torch

from aici_b200 import _lib, tch_cuda
from aici_b200._lib import AiciError
from oracle import cpu_oracle as O

pytestmark = pytest.mark.gpu
REF_LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref",
                       "libref_vllm.so")


def _cache(nblk, hkv, seed, value=False):
    g = torch.Generator().manual_seed(seed)
    shape = (nblk, hkv, 128, 16) if value else (nblk, hkv, 16, 16, 8)
    return torch.randn(shape, generator=g).to(torch.bfloat16)


def _mapping(n_src, n_dst, pairs, seed):
    g = torch.Generator().manual_seed(seed)
    src = torch.randperm(n_src, generator=g)[:pairs].tolist()
    dst = torch.randperm(n_dst, generator=g)[:pairs].tolist()
    return dict(zip(src, dst))


def _same(a, b):
    return torch.equal(a.cpu().contiguous().view(torch.int16), b.cpu().contiguous().view(torch.int16))


@pytest.mark.parametrize("pinned", [True, False])
@pytest.mark.parametrize("hkv,pairs,value", [(8, 1, False), (8, 37, True), (32, 200, False), (1, 64, True)])
def test_swap_out_then_in_round_trip(cuda_device, pinned, hkv, pairs, value):
    n_gpu, n_cpu = 256, 300
    gpu0 = _cache(n_gpu, hkv, 1, value)
    cpu0 = _cache(n_cpu, hkv, 2, value)
    gpu = gpu0.to(cuda_device)
    host = cpu0.clone().pin_memory() if pinned else cpu0.clone()
    out_map = _mapping(n_gpu, n_cpu, pairs, 3)

    # swap out: device -> host, against the oracle
    want_host = cpu0.clone()
    O.swap_blocks(gpu0, want_host, out_map)
    tch_cuda.swap_blocks(gpu, host, out_map)
    torch.cuda.synchronize()
    assert _same(host, want_host)
    assert _same(gpu, gpu0)  # the source is untouched

    # poison the swapped-out device blocks, then swap in: host -> device
    for s in out_map:
        gpu[s].fill_(float("nan"))
    in_map = {d: s for s, d in out_map.items()}
    tch_cuda.swap_blocks(host, gpu, in_map)
    torch.cuda.synchronize()
    assert _same(gpu, gpu0)
    assert _lib.last_status() == 0


def test_flat_mapping_with_runs_and_many_pairs(cuda_device):
    """More pairs than one launch carries, consecutive runs (merged on the pageable path) and a
    flat int64 tensor instead of a dict."""
    n = 4000
    gpu0 = _cache(n, 2, 5)
    gpu = gpu0.to(cuda_device)
    src = torch.arange(0, n, dtype=torch.int64)
    dst = torch.cat([torch.arange(100, n, dtype=torch.int64), torch.arange(0, 100, dtype=torch.int64)])
    pairs = torch.stack([src, dst], 1).reshape(-1)
    want = torch.empty_like(gpu0)
    O.swap_blocks(gpu0, want, pairs.tolist())
    for host in (torch.zeros_like(gpu0).pin_memory(), torch.zeros_like(gpu0)):
        tch_cuda.swap_blocks(gpu, host, pairs)
        torch.cuda.synchronize()
        assert _same(host, want)


def test_device_to_device(cuda_device):
    a0, b0 = _cache(128, 8, 7, True), _cache(96, 8, 8, True)
    a, b = a0.to(cuda_device), b0.to(cuda_device)
    m = _mapping(128, 96, 50, 9)
    want = b0.clone()
    O.swap_blocks(a0, want, m)
    tch_cuda.swap_blocks(a, b, m)
    torch.cuda.synchronize()
    assert _same(b, want) and _same(a, a0)


def test_empty_mapping_and_errors(cuda_device):
    gpu = _cache(8, 1, 1).to(cuda_device)
    host = _cache(8, 1, 2)
    tch_cuda.swap_blocks(gpu, host, {})
    with pytest.raises(AiciError, match="Invalid device combination"):
        tch_cuda.swap_blocks(host, host.clone(), {0: 1})
    with pytest.raises(AiciError, match="outside the cache"):
        tch_cuda.swap_blocks(gpu, host, {8: 0})
    with pytest.raises(AiciError, match="outside the cache"):
        tch_cuda.swap_blocks(gpu, host, {0: 8})
    with pytest.raises(AiciError, match="same block shape"):
        tch_cuda.swap_blocks(gpu, _cache(8, 2, 2), {0: 1})
    assert _lib.last_status() == 0


def _ref_swap(ref, src, dst, mapping):
    pairs = torch.tensor([x for s_, d_ in mapping.items() for x in (s_, d_)], dtype=torch.int64)
    dev = lambda t: t.device.index if t.is_cuda else -1
    res = ref.ref_swap_blocks(ctypes.c_void_p(src.data_ptr()), dev(src), ctypes.c_void_p(dst.data_ptr()), dev(dst),
                              ctypes.c_void_p(pairs.data_ptr()), ctypes.c_int64(len(mapping)),
                              ctypes.c_int64(src.shape[0]), ctypes.c_int64(dst.shape[0]),
                              ctypes.c_int64(src[0].numel()))
    assert not res, ctypes.string_at(res)
    torch.cuda.synchronize()


@pytest.mark.parametrize("direction", ["device_to_pinned", "pinned_to_device", "device_to_pageable",
                                       "pageable_to_device", "device_to_device"])
@pytest.mark.parametrize("hkv,pairs,value", [(8, 37, True), (32, 150, False)])
def test_bit_exact_vs_reference_swap_blocks(cuda_device, direction, hkv, pairs, value):
    """Ours and the reference's own function on identical inputs: destinations must agree bit for bit
    (every block, the untouched ones included) and sources must stay as they were."""
    if not os.path.exists(REF_LIB):
        pytest.skip("reference comparator not built (python oracle/build_ref.py)")
    ref = ctypes.CDLL(REF_LIB)
    if not hasattr(ref, "ref_swap_blocks"):
        pytest.skip("comparator library predates ref_swap_blocks: rebuild it (python oracle/build_ref.py --force)")
    ref.ref_swap_blocks.restype = ctypes.c_void_p
    n_src, n_dst = 200, 260
    src0, dst0 = _cache(n_src, hkv, 11, value), _cache(n_dst, hkv, 12, value)
    src_kind, dst_kind = direction.split("_to_")

    def place(t, kind):
        if kind == "device":
            return t.to(cuda_device)
        return t.clone().pin_memory() if kind == "pinned" else t.clone()
    m = _mapping(n_src, n_dst, pairs, 13)
    src_a, dst_a = place(src0, src_kind), place(dst0, dst_kind)
    src_b, dst_b = place(src0, src_kind), place(dst0, dst_kind)
    tch_cuda.swap_blocks(src_a, dst_a, m)
    torch.cuda.synchronize()
    _ref_swap(ref, src_b, dst_b, m)
    assert _same(dst_a, dst_b)
    assert _same(src_a, src0) and _same(src_b, src0)
    assert not _same(dst_a, dst0)
    assert _lib.last_status() == 0


def test_cache_on_another_gpu_than_the_current_one_is_refused():
    """The copy kernel runs on the current device, so a cache that lives elsewhere is an error
    (through the raw C ABI: the Python mirror would make the cache's GPU current itself)."""
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    torch.cuda.set_device(0)
    gpu1 = _cache(8, 1, 1).to("cuda:1")
    host = _cache(8, 1, 2).pin_memory()
    pairs = torch.tensor([0, 1], dtype=torch.int64)
    res = _lib.lib().aici_swap_blocks(ctypes.c_void_p(gpu1.data_ptr()), ctypes.c_void_p(host.data_ptr()),
                                      ctypes.c_void_p(pairs.data_ptr()), 1, ctypes.c_int64(gpu1[0].numel() * 2),
                                      ctypes.c_int64(8), ctypes.c_int64(8), None)
    with pytest.raises(AiciError, match="current device"):
        _lib.check("swap_blocks", res)
