"""ctypes view of ``libfastgl_b200.so`` (the C ABI declared in include/fastgl_b200.h).

Loading needs no GPU; the first call that touches the device creates a workspace.  A missing
library is an ImportError: there is no other implementation behind the ``fastgl`` ops.
"""
from __future__ import annotations

import ctypes
import os

MAX_HOPS = 7
COUNTS_STRIDE = 16
AGG_SUM, AGG_MEAN, AGG_SYMNORM = 0, 1, 2
FLAG_SAMPLE_REPLACE = 1
FLAG_MAP_ARRIVAL_ORDER = 2
FLAG_ZERO_DEG_PASSTHROUGH = 1
ABI_VERSION = 3

# FASTGL_B200_LIB points at another build of the same library (kernel experiments)
LIB_PATH = os.environ.get("FASTGL_B200_LIB") or os.path.join(os.path.dirname(os.path.abspath(__file__)), "libfastgl_b200.so")

# every symbol include/fastgl_b200.h declares
EXPORTS = (
    "fgl_abi_version", "fgl_sizeof_fused_args", "fgl_status_str", "fgl_ws_create", "fgl_ws_destroy", "fgl_ws_reserve", "fgl_last_error",
    "fgl_ws_check", "fgl_ws_status_peek", "fgl_ws_time_next_launch", "fgl_selftest_barrier_timeout", "fgl_probe_access_pattern", "fgl_sample", "fgl_map", "fgl_fused_capacity", "fgl_sample_map_fused", "fgl_cal_deg",
    "fgl_stage_segments", "fgl_window_overlap", "fgl_exclusive_sum", "fgl_exclusive_sum_noalloc", "fgl_exclusive_sum_noalloc_status", "fgl_agg_fwd", "fgl_agg_fwd_sharded", "fgl_gather_rows", "fgl_agg_edge_fwd", "fgl_agg_edge_bwd", "fgl_agg_edge_wgrad", "fgl_agg_fwd_window", "fgl_agg_bwd",
    "fgl_agg_bwd_self", "fgl_block_transpose", "fgl_agg_bwd_gather", "fgl_bias_relu_dropout", "fgl_relu_dropout_bwd", "fgl_relu_dropout_bwd_split", "fgl_softmax_xent", "fgl_linear_softmax_xent", "fgl_adam_step", "fgl_split_tf32", "fgl_fold_blocks",
    "fgl_sizeof_peer_sync", "fgl_peer_sync_chunks", "fgl_allreduce_adam",
)


class FusedArgs(ctypes.Structure):
    """struct fgl_fused_args"""
    _fields_ = [
        ("indptr", ctypes.c_void_p),
        ("indices", ctypes.c_void_p),
        ("n_nodes", ctypes.c_int64),
        ("indptr_is_64", ctypes.c_int32),
        ("n_batches", ctypes.c_int32),
        ("n_hops", ctypes.c_int32),
        ("fanout", ctypes.c_int32 * MAX_HOPS),
        ("flags", ctypes.c_int32),
        ("n_teams", ctypes.c_int32),
        ("table_slots_hint", ctypes.c_int64),
        ("rng_seed", ctypes.c_uint64),
        ("rng_ctr", ctypes.c_uint64),
        ("seeds", ctypes.c_void_p),
        ("seed_stride", ctypes.c_int64),
        ("seed_counts", ctypes.c_void_p),
        ("nodes", ctypes.c_void_p),
        ("nodes_stride", ctypes.c_int64),
        ("counts", ctypes.c_void_p),
        ("block_indptr", ctypes.c_void_p * MAX_HOPS),
        ("block_indptr_stride", ctypes.c_int64 * MAX_HOPS),
        ("block_src", ctypes.c_void_p * MAX_HOPS),
        ("block_src_stride", ctypes.c_int64 * MAX_HOPS),
    ]


MAX_PEERS = 8


class PeerSync(ctypes.Structure):
    """struct fgl_peer_sync"""
    _fields_ = [("rank", ctypes.c_int32), ("world", ctypes.c_int32), ("recv", ctypes.c_void_p * MAX_PEERS),
                ("flags", ctypes.c_void_p * MAX_PEERS), ("n_pad", ctypes.c_int64), ("n_chunks", ctypes.c_int32)]


class Segment(ctypes.Structure):
    """struct fgl_segment"""
    _fields_ = [("dst", ctypes.c_void_p), ("src", ctypes.c_void_p), ("bytes", ctypes.c_int64)]


MAX_SEGMENTS = 8

_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `make -C fastgl-ae_b200/csrc` (nvcc, sm_100a). "
                "The fastgl ops have no CPU or PyTorch fallback.")
        handle = ctypes.CDLL(LIB_PATH)
        missing = [s for s in EXPORTS if not hasattr(handle, s)]
        if missing:
            raise ImportError(f"{LIB_PATH} lacks symbols {missing}")
        handle.fgl_abi_version.restype = ctypes.c_int
        if handle.fgl_abi_version() != ABI_VERSION:
            raise ImportError(f"{LIB_PATH}: ABI version {handle.fgl_abi_version()} != {ABI_VERSION}")
        if handle.fgl_sizeof_fused_args() != ctypes.sizeof(FusedArgs):
            raise ImportError("struct fgl_fused_args layout differs between the library and this binding")
        handle.fgl_status_str.restype = ctypes.c_char_p
        handle.fgl_status_str.argtypes = [ctypes.c_int]
        handle.fgl_last_error.restype = ctypes.c_char_p
        handle.fgl_last_error.argtypes = [ctypes.c_void_p]
        for name in EXPORTS:
            if name not in ("fgl_status_str", "fgl_last_error"):
                getattr(handle, name).restype = ctypes.c_int
        handle.fgl_peer_sync_chunks.restype = ctypes.c_int64
        handle.fgl_peer_sync_chunks.argtypes = [ctypes.c_int64]
        if handle.fgl_sizeof_peer_sync() != ctypes.sizeof(PeerSync):
            raise ImportError("struct fgl_peer_sync layout differs between the library and this binding")
        _lib = handle
    return _lib


def status_str(rc: int) -> str:
    return lib().fgl_status_str(rc).decode()


lib()
