"""CPU checks of the boundary: the library builds, loads and exports exactly what the header
declares; host-side argument checks reject what the reference rejects.  No kernel runs here."""
import ctypes
import os
import re
import subprocess

import pytest
import torch

import aici_b200
from aici_b200 import _lib, build, tch_cuda
import workloads
from aici_b200._lib import AiciError

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def built_lib():
    return build.build()


def _header_symbols():
    text = open(os.path.join(ROOT, "include", "aici_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(aici_[a-z0-9_]+)\s*\(", text)))


def test_header_matches_loader_list():
    assert _header_symbols() == sorted(_lib.EXPORTS)


def test_library_exports_every_declared_symbol(built_lib):
    lib = ctypes.CDLL(built_lib)
    for name in _header_symbols():
        assert hasattr(lib, name), name
    out = subprocess.run(["nm", "-D", "--defined-only", built_lib], capture_output=True, text=True).stdout
    for name in _header_symbols():
        assert re.search(r"\bT %s\b" % name, out), name


def test_library_has_no_torch_or_python_dependency(built_lib):
    out = subprocess.run(["ldd", built_lib], capture_output=True, text=True).stdout
    assert "torch" not in out and "python" not in out and "c10" not in out


def test_version_and_error_convention(built_lib):
    lib = _lib.lib()
    assert b"sm_100a" in lib.aici_version()
    # host-side validation happens before any CUDA call: unsupported head size -> error string
    res = lib.aici_reshape_and_cache(None, None, None, None, None, 0, 4, 2, 64, 16,
                                     ctypes.c_int64(8), ctypes.c_int64(128), ctypes.c_int64(128), 0, None)
    with pytest.raises(AiciError, match="head_size must be 128"):
        _lib.check("reshape_and_cache", res)
    res = lib.aici_paged_attention_v1(None, None, None, None, 3, ctypes.c_float(1.0), None, None, 16, 64,
                                      None, 1, 8, 128, 4, ctypes.c_int64(8), ctypes.c_int64(1024),
                                      ctypes.c_int64(1), ctypes.c_int64(1), None, ctypes.c_size_t(0), 0, None)
    with pytest.raises(AiciError, match="not divisible"):
        _lib.check("paged_attention_v1", res)
    res = lib.aici_mha_varlen_fwd(None, None, None, None, None, None, 0, 0, 0, 1, 1, 128, 0, 0,
                                  *[ctypes.c_int64(128)] * 8, ctypes.c_float(1.0), 1, 0, None)
    with pytest.raises(AiciError, match="batch size must be positive"):
        _lib.check("flash_attn_varlen", res)
    res = lib.aici_copy_blocks_host(None, None, None, 0, 0, ctypes.c_int64(0), ctypes.c_int64(0), 0, None)
    with pytest.raises(AiciError, match="multiple of 16 bytes"):
        _lib.check("copy_blocks", res)
    # one fp32 partial (128 values + max + sum) per piece; pieces < warps of the grid + rows
    need = lib.aici_paged_attention_workspace_bytes(64, 32, 32, 4096)
    assert 64 * 32 * 130 * 4 < need < (64 * 32 + 4 * 2 * 256) * 132 * 4


def test_argument_checks_of_the_multi_gpu_entry_points(built_lib):
    """Host-side validation only (pointers are never dereferenced before these checks fail)."""
    lib = _lib.lib()
    fake = ctypes.c_void_p(0x10000)
    outs = (ctypes.c_void_p * 2)(fake, fake)
    i64 = ctypes.c_int64
    # this rank's heads [6, 10) do not fit an 8-head output row
    res = lib.aici_mha_varlen_fwd_peers(outs, 2, 6, fake, fake, fake, fake, fake, 1, 128, 128, 4, 4, 128, 128, 128,
                                        i64(512), i64(128), i64(512), i64(128), i64(512), i64(128), i64(1024),
                                        i64(128), ctypes.c_float(0.1), 1, 0, None)
    with pytest.raises(AiciError, match="do not fit an output row"):
        _lib.check("flash_attn_varlen_peers", res)
    res = lib.aici_paged_attention_v1_peers_barrier(outs, outs, 2, 2, 8, 0, *[None] * 3, 4, ctypes.c_float(1.0),
                                                    None, None, 16, 64, 1, 4, 128, 4, i64(8), i64(512), i64(1),
                                                    i64(1), None, ctypes.c_size_t(0), 0, None)
    with pytest.raises(AiciError, match="rank inside it"):
        _lib.check("paged_attention_v1_peers_barrier", res)
    res = lib.aici_gather_heads(outs, 2, 8, 6, fake, i64(4), 4, 128, i64(512), 0, None)
    with pytest.raises(AiciError, match="do not fit 8 total heads"):
        _lib.check("gather_heads", res)
    res = lib.aici_peer_open(None, None)
    with pytest.raises(AiciError, match="NULL pointer"):
        _lib.check("peer_open", res)
    bogus = (ctypes.c_ubyte * 128)()
    out = ctypes.c_void_p(0)
    res = lib.aici_peer_open(bogus, ctypes.byref(out))
    with pytest.raises(AiciError, match="not a handle made by aici_peer_alloc"):
        _lib.check("peer_open", res)
    res = lib.aici_mha_varlen_fwd_shape(fake, fake, fake, fake, fake, fake, 1, 128, 128, 4, 4, 128, 128, 128,
                                        *[i64(512), i64(128)] * 4, ctypes.c_float(0.1), 1, 3, 0, None)
    with pytest.raises(AiciError, match="multiple of 4"):
        _lib.check("flash_attn_varlen", res)
    assert lib.aici_paged_attention_chunked_workspace_bytes(64, 32, 32, 4096, 24) == 256  # invalid chunk size


def test_product_path_refuses_cpu_tensors():
    k = torch.zeros(1, 2, 128, dtype=torch.bfloat16)
    kc = torch.zeros(2, 2, 16, 16, 8, dtype=torch.bfloat16)
    vc = torch.zeros(2, 2, 128, 16, dtype=torch.bfloat16)
    with pytest.raises(AiciError, match="no CPU path"):
        tch_cuda.reshape_and_cache(k, k, kc, vc, torch.zeros(1, dtype=torch.int32))
    with pytest.raises(AiciError, match="no CPU path"):
        tch_cuda.copy_blocks([kc], [vc], {0: [1]})
    with pytest.raises(AiciError, match="no CPU path"):
        tch_cuda.flash_attn_varlen(k, k, k, torch.zeros(2, dtype=torch.int32),
                                   torch.zeros(2, dtype=torch.int32), 1, 1, 1.0, True)


def test_product_package_does_not_import_oracle():
    for root, _dirs, files in os.walk(os.path.dirname(aici_b200.__file__)):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(root, f)).read()
                assert "oracle" not in text, os.path.join(root, f)


def test_workload_generators_shapes_and_bytes():
    w = workloads.make_decode("t", "cpu", num_seqs=5, num_heads=8, num_kv_heads=2, ctx_kind="uniform",
                              ctx_lo=3, ctx_hi=70, pool_blocks=64, seed=1)
    assert w.key_cache.shape == (64, 2, 16, 16, 8) and w.value_cache.shape == (64, 2, 128, 16)
    assert w.block_tables.shape[0] == 5 and w.max_context_len == max(w.context_list)
    used = set()
    for i, c in enumerate(w.context_list):
        row = w.block_tables[i, :(c + 15) // 16].tolist()
        assert not (used & set(row))
        used |= set(row)
        assert int(w.slot_mapping[i]) == row[(c - 1) // 16] * 16 + (c - 1) % 16
    kv = sum(w.context_list) * 2 * 2 * 128 * 2
    assert w.algorithmic_bytes() > kv and w.algorithmic_bytes() < kv * 1.2 + 10000
    ws = workloads.make_decode("t", "cpu", num_seqs=5, num_heads=8, num_kv_heads=2, ctx_kind="uniform",
                               ctx_lo=3, ctx_hi=70, pool_blocks=64, seed=1,
                               shard=workloads.Shard(rank=1, world=2))
    assert torch.equal(ws.key_cache, w.key_cache[:, 1:2]) and torch.equal(ws.query, w.query[:, 4:8])
    ctx = workloads.draw_context_lens("loguniform", 1000, 128, 8192, 5)
    assert min(ctx) >= 128 and max(ctx) <= 8192 and 1500 < sum(ctx) / 1000 < 2400
    p = workloads.make_prefill("p", "cpu", lens_q=[4, 9], lens_k=[6, 9], num_heads=4, num_kv_heads=2, seed=3)
    assert p.cu_seqlens_q.tolist() == [0, 4, 13] and p.cu_seqlens_k.tolist() == [0, 6, 15]
    assert p.flops() == 4.0 * 128 * 4 * ((4 * 2 + 10) + 45)
    m = workloads.fork_block_mapping([[1, 2], [3]], 2, 2, [10, 11, 12, 13])
    assert m == {2: [10, 11], 3: [12, 13]}
