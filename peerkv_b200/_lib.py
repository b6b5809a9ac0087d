"""ctypes binding of libpeerkv.so, the C-ABI CUDA library (include/peerkv.h).

There is no fallback: if the library is missing or fails to load, every entry
point of the package raises.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libpeerkv.so")

PKV_F16, PKV_BF16, PKV_INT8, PKV_FP8_E4M3, PKV_F32 = 0, 1, 2, 3, 4
ST_PIPE_TIMEOUT, ST_BAD_PAGE, ST_Q_TIMEOUT, ST_PARTIAL_TIMEOUT = 1, 2, 4, 8

EXPORTS = [
    "pkv_last_error", "pkv_abi_version", "pkv_shard_create", "pkv_shard_destroy",
    "pkv_shard_status", "pkv_decode_partial", "pkv_decode", "pkv_decode_static", "pkv_decode_splits_only", "pkv_merge_partials",
    "pkv_quantize_kv", "pkv_split_block_table", "pkv_exchange_create", "pkv_exchange_destroy", "pkv_exchange_export",
    "pkv_exchange_import", "pkv_exchange_attach", "pkv_exchange_status", "pkv_exchange_epoch",
    "pkv_home_publish_q", "pkv_home_step", "pkv_peer_step", "pkv_home_partial", "pkv_home_merge",
    "pkv_static_status", "pkv_shard_trace", "pkv_exchange_resync", "pkv_exchange_capture_begin",
    "pkv_exchange_capture_end", "pkv_exchange_replayed",
    "pkv_add_rmsnorm", "pkv_rope_append", "pkv_swiglu", "pkv_kv_append",
    "pkv_enable_peer_access", "pkv_shard_stats", "pkv_prefill_partial", "pkv_stage_peer_blocks",
    "pkv_exchange_hop_probe", "pkv_exchange_hop_probe_reset",
]


class KvView(C.Structure):
    _fields_ = [("k", C.c_void_p), ("v", C.c_void_p), ("k_scale", C.c_void_p),
                ("v_scale", C.c_void_p), ("dtype", C.c_int32), ("n_kv_heads", C.c_int32),
                ("head_dim", C.c_int32), ("page_size", C.c_int32), ("n_pages", C.c_int64),
                ("page_stride", C.c_int64), ("token_stride", C.c_int64),
                ("head_stride", C.c_int64)]


class DecodeArgs(C.Structure):
    _fields_ = [("q", C.c_void_p), ("q_dtype", C.c_int32), ("batch", C.c_int32),
                ("n_q_heads", C.c_int32), ("reserved0", C.c_int32), ("kv", KvView),
                ("block_table", C.c_void_p), ("block_table_stride", C.c_int64),
                ("seq_lens", C.c_void_p), ("scale", C.c_float), ("reserved1", C.c_int32)]


class PeerKVError(RuntimeError):
    pass


_lib = None


def lib():
    """The loaded library; raises if it was not built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise PeerKVError(
            f"{LIB_PATH} is missing: build it with `python -m peerkv_b200.build` "
            "(the package has no CPU or PyTorch fallback)")
    L = C.CDLL(LIB_PATH)
    for name in EXPORTS:
        if not hasattr(L, name):
            raise PeerKVError(f"{LIB_PATH} does not export {name}")
    L.pkv_last_error.restype = C.c_char_p
    vp, i32, i64, u32, u64, f32 = C.c_void_p, C.c_int32, C.c_int64, C.c_uint32, C.c_uint64, C.c_float
    P = C.POINTER
    sig = {
        "pkv_abi_version": [],
        "pkv_shard_create": [P(vp), C.c_int, C.c_int, C.c_int],
        "pkv_shard_destroy": [vp],
        "pkv_shard_status": [vp, vp, P(u32)],
        "pkv_decode_partial": [vp, P(DecodeArgs), vp, vp, vp],
        "pkv_decode": [vp, P(DecodeArgs), vp, i32, vp, vp],
        "pkv_decode_static": [C.c_int, P(DecodeArgs), vp, i32, vp, vp],
        "pkv_decode_splits_only": [vp, P(DecodeArgs), vp],
        "pkv_merge_partials": [C.c_int, vp, i64, vp, i64, i32, i32, i32, vp, i32, vp, vp],
        "pkv_quantize_kv": [C.c_int, vp, i32, i64, vp, vp, i32, vp],
        "pkv_split_block_table": [C.c_int, vp, i64, vp, i32, i32, i32, i32, P(i64), P(vp), i64, P(vp), vp],
        "pkv_exchange_create": [P(vp), C.c_int, C.c_int, C.c_int, C.c_int, C.c_int],
        "pkv_exchange_destroy": [vp],
        "pkv_exchange_export": [vp, vp],
        "pkv_exchange_import": [vp, C.c_int, vp],
        "pkv_exchange_attach": [vp, C.c_int, vp],
        "pkv_exchange_status": [vp, vp, P(u32)],
        "pkv_exchange_epoch": [vp, P(u64)],
        "pkv_home_publish_q": [vp, vp, i32, vp],
        "pkv_home_step": [vp, vp, P(DecodeArgs), u32, vp, i32, vp, vp],
        "pkv_peer_step": [vp, vp, P(DecodeArgs), i32, i32, vp],
        "pkv_home_partial": [vp, vp, P(DecodeArgs), vp],
        "pkv_home_merge": [vp, i32, u32, vp, i32, vp, vp],
        "pkv_static_status": [C.c_int, vp, P(u32)],
        "pkv_shard_trace": [vp, vp],
        "pkv_exchange_resync": [vp, u64],
        "pkv_exchange_capture_begin": [vp],
        "pkv_exchange_capture_end": [vp, vp, P(u64)],
        "pkv_exchange_replayed": [vp],
        "pkv_add_rmsnorm": [C.c_int, vp, vp, vp, vp, i32, i32, f32, i32, vp],
        "pkv_rope_append": [C.c_int, vp, vp, vp, i32, i32, i32, i32, vp, vp, vp, i64, i64, i64, vp, vp, i32, vp],
        "pkv_swiglu": [C.c_int, vp, vp, i32, i32, i32, vp],
        "pkv_enable_peer_access": [C.c_int, C.c_int],
        "pkv_shard_stats": [vp, vp, P(u64), P(u64)],
        "pkv_stage_peer_blocks": [C.c_int, vp, i64, vp, i32, i32, i32, P(i64), P(i64), P(vp), P(vp), P(i64), vp, vp,
                                  i64, i64, i64, i64, i32, vp, vp, vp, vp],
        "pkv_exchange_hop_probe": [vp, i32, i32, i32, i32, vp, vp],
        "pkv_exchange_hop_probe_reset": [vp, vp],
        "pkv_prefill_partial": [C.c_int, vp, i64, i64, i64, vp, vp, i64, i64, i64, i32, i32, i32, i32, i32, i32, i32,
                                f32, i32, i64, i64, vp, vp, vp],
        "pkv_kv_append": [C.c_int, vp, vp, i64, vp, i32, i32, i32, i32, i32, P(i64), P(i64), P(vp), P(vp),
                          P(i64), P(i64), P(i64), vp, vp],
    }
    for name, args in sig.items():
        fn = getattr(L, name)
        fn.argtypes = args
        fn.restype = C.c_int
    if L.pkv_abi_version() != 1:
        raise PeerKVError("libpeerkv.so ABI version mismatch; rebuild it")
    _lib = L
    return L


def check(rc: int):
    if rc != 0:
        raise PeerKVError(f"peerkv error {rc}: {lib().pkv_last_error().decode()}")
