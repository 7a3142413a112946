"""Loads libaici_b200.so (the C ABI of include/aici_b200.h) through ctypes.

There is no CPU or PyTorch fallback: if the library is missing, or a call returns an error
string, the caller gets an exception.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libaici_b200.so")

# Every symbol include/aici_b200.h declares (the CPU test-suite checks this list against
# the header and against the built library).
EXPORTS = (
    "aici_version",
    "aici_last_status",
    "aici_reshape_and_cache",
    "aici_gather_cached_kv",
    "aici_rotary_reshape_and_cache",
    "aici_copy_blocks",
    "aici_copy_blocks_host",
    "aici_paged_attention_workspace_bytes",
    "aici_paged_attention_chunked_workspace_bytes",
    "aici_paged_attention_v1_chunked",
    "aici_paged_attention_v1",
    "aici_paged_attention_v2",
    "aici_paged_attention_v1_static",
    "aici_mha_varlen_fwd",
    "aici_mha_varlen_fwd_shape",
    "aici_mha_varlen_paged_fwd",
    "aici_paged_attention_v1_peers",
    "aici_mha_varlen_fwd_peers",
    "aici_peer_barrier",
    "aici_paged_attention_v1_peers_barrier",
    "aici_decode_step",
    "aici_peer_alloc",
    "aici_peer_open",
    "aici_peer_close",
    "aici_peer_free",
    "aici_gather_heads",
    "aici_swap_blocks",
    "aici_batch_info_layout",
    "aici_batch_info_build",
)

_lib = None


class AiciError(RuntimeError):
    """An entry point returned a non-NULL error string (the reference panics here,
    rllm/tch-cuda/src/lib.rs:22-27)."""


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise AiciError(
                "libaici_b200.so is not built: run `python -m aici_b200.build` "
                "(nvcc, sm_100a). There is no fallback path.")
        _lib = ctypes.CDLL(LIB_PATH)
        _lib.aici_version.restype = ctypes.c_char_p
        _lib.aici_paged_attention_workspace_bytes.restype = ctypes.c_size_t
        _lib.aici_paged_attention_chunked_workspace_bytes.restype = ctypes.c_size_t
        for name in EXPORTS:
            fn = getattr(_lib, name)
            if name not in ("aici_version", "aici_paged_attention_workspace_bytes",
                            "aici_paged_attention_chunked_workspace_bytes"):
                fn.restype = ctypes.c_void_p  # char*, released with free()
        _libc = ctypes.CDLL(None)
        _libc.free.argtypes = [ctypes.c_void_p]
        _lib._free = _libc.free
    return _lib


def check(fn_name: str, res) -> None:
    """NULL = ok; otherwise raise with the message and free() it."""
    if res:
        msg = ctypes.string_at(res).decode("utf-8", "replace")
        lib()._free(res)
        raise AiciError("%s: %s" % (fn_name, msg))


def last_status() -> int:
    out = ctypes.c_int(0)
    check("aici_last_status", lib().aici_last_status(ctypes.byref(out)))
    return out.value
