"""GPU parity tests (bit-exact) for swap_blocks through the C ABI: device <-> page-locked host
(kernel over PCIe), device <-> pageable host (copy engine), device <-> device."""
import pytest
import torch

from aici_b200 import _lib, tch_cuda
from aici_b200._lib import AiciError
from oracle import cpu_oracle as O

pytestmark = pytest.mark.gpu


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
