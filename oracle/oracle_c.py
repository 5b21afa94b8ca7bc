"""ctypes binding of the C oracle (``fgl_oracle.c``).  Test infrastructure only.

Used by the tests, the smoke check and the CPU-baseline leg of the benchmark;
the shipped package never imports it.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libfgl_oracle.so")
_lib = None

MODE_SUM, MODE_MEAN, MODE_SYMNORM = 0, 1, 2


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "fgl_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "libfgl_oracle.so"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.fglo_sample.restype = ctypes.c_int64
        _lib.fglo_map.restype = ctypes.c_int64
        _lib.fglo_max_threads.restype = ctypes.c_int
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _i32(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.int32)


def max_threads() -> int:
    return int(lib().fglo_max_threads())


def set_threads(n: int) -> None:
    lib().fglo_set_threads(ctypes.c_int(n))


def philox4x32_10(ctr, key):
    c = np.asarray(ctr, dtype=np.uint32)
    k = np.asarray(key, dtype=np.uint32)
    out = np.zeros(4, dtype=np.uint32)
    lib().fglo_philox4x32_10(_p(c), _p(k), _p(out))
    return tuple(int(v) for v in out)


def sample(indptr, indices, seeds, fanout, replace=False, rng_seed=0, rng_ctr=0):
    indptr = np.ascontiguousarray(indptr, dtype=np.int64)
    indices = _i32(indices)
    seeds = _i32(seeds)
    S = seeds.shape[0]
    out_ptr = np.zeros(S + 1, dtype=np.int32)
    out_src = np.zeros(max(1, S * fanout), dtype=np.int32)
    out_dst = np.zeros(max(1, S * fanout), dtype=np.int32)
    E = lib().fglo_sample(_p(indptr), _p(indices), _p(seeds), ctypes.c_int32(S), ctypes.c_int32(fanout),
                          ctypes.c_int(int(replace)), ctypes.c_uint64(rng_seed), ctypes.c_uint64(rng_ctr),
                          _p(out_ptr), _p(out_src), _p(out_dst))
    return out_ptr, out_src[:E].copy(), out_dst[:E].copy()


def map_edges(src_global, dst_global, seeds):
    src = _i32(src_global).copy()
    dst = _i32(dst_global).copy()
    seeds = _i32(seeds)
    S, E = seeds.shape[0], src.shape[0]
    unique = np.zeros(max(1, S + E), dtype=np.int32)
    U = lib().fglo_map(_p(src), _p(dst), _p(seeds), ctypes.c_int32(S), ctypes.c_int64(E), _p(unique))
    return src, dst, unique[:U].copy()


def sample_blocks(indptr, indices, seeds, fanouts, replace=False, rng_seed=0, rng_ctr=0):
    """Multi-hop loop of FusedMapSampler.sample_blocks (FusedMapSampler.py:63-109); blocks input-layer first."""
    seeds = _i32(seeds)
    cur = seeds
    blocks = []
    for h, fanout in enumerate(reversed(list(fanouts))):
        ptr, src_g, dst_g = sample(indptr, indices, cur, fanout, replace, rng_seed, rng_ctr + h)
        src_l, dst_l, uniq = map_edges(src_g, dst_g, cur)
        blocks.insert(0, dict(indptr=ptr, src_local=src_l, dst_local=dst_l,
                              n_src=int(uniq.shape[0]), n_dst=int(cur.shape[0])))
        cur = uniq
    return cur, seeds, blocks


def cal_deg(ids, nodes_num):
    ids = _i32(ids)
    deg = np.zeros(nodes_num, dtype=np.int32)
    lib().fglo_cal_deg(_p(ids), ctypes.c_int64(ids.shape[0]), ctypes.c_int32(nodes_num), _p(deg))
    return deg


def exclusive_sum(degs):
    degs = _i32(degs)
    out = np.zeros(degs.shape[0] + 1, dtype=np.int32)
    lib().fglo_exclusive_sum(_p(degs), ctypes.c_int64(degs.shape[0]), _p(out))
    return out


def aggregate_fwd(mode, indptr, src, x, n_dst, src_deg=None, dst_deg=None, zero_deg_passthrough=True,
                  row_map=None):
    x = np.ascontiguousarray(x, dtype=np.float32)
    indptr, src = _i32(indptr), _i32(src)
    src_deg, dst_deg, row_map = _i32(src_deg), _i32(dst_deg), _i32(row_map)
    D = x.shape[1]
    out = np.zeros((n_dst, D), dtype=np.float32)
    lib().fglo_agg_fwd(ctypes.c_int(mode), _p(indptr), _p(src), _p(src_deg), _p(dst_deg), _p(row_map), _p(x),
                       ctypes.c_int64(D), ctypes.c_int32(D), ctypes.c_int32(n_dst),
                       ctypes.c_int(int(zero_deg_passthrough)), _p(out), ctypes.c_int64(D))
    return out


def aggregate_bwd(mode, indptr, src, dy, n_src, src_deg=None, dst_deg=None):
    dy = np.ascontiguousarray(dy, dtype=np.float32)
    indptr, src = _i32(indptr), _i32(src)
    src_deg, dst_deg = _i32(src_deg), _i32(dst_deg)
    n_dst, D = dy.shape
    dx = np.zeros((n_src, D), dtype=np.float32)
    lib().fglo_agg_bwd(ctypes.c_int(mode), _p(indptr), _p(src), _p(src_deg), _p(dst_deg), _p(dy),
                       ctypes.c_int64(D), ctypes.c_int32(D), ctypes.c_int32(n_dst), ctypes.c_int32(n_src),
                       _p(dx), ctypes.c_int64(D))
    return dx


def aggregate_edge_fwd(indptr, src, edge_w, x, n_dst, zero_deg_passthrough=True):
    x = np.ascontiguousarray(x, dtype=np.float32)
    edge_w = np.ascontiguousarray(edge_w, dtype=np.float32)
    indptr, src = _i32(indptr), _i32(src)
    D, H = x.shape[1], edge_w.shape[1]
    out = np.zeros((n_dst, D), dtype=np.float32)
    lib().fglo_agg_edge_fwd(_p(indptr), _p(src), _p(edge_w), ctypes.c_int32(H), _p(x), ctypes.c_int64(D), ctypes.c_int32(D),
                            ctypes.c_int32(n_dst), ctypes.c_int(int(zero_deg_passthrough)), _p(out), ctypes.c_int64(D))
    return out


def aggregate_edge_bwd(indptr, src, edge_w, dy, n_src):
    dy = np.ascontiguousarray(dy, dtype=np.float32)
    edge_w = np.ascontiguousarray(edge_w, dtype=np.float32)
    indptr, src = _i32(indptr), _i32(src)
    n_dst, D = dy.shape
    dx = np.zeros((n_src, D), dtype=np.float32)
    lib().fglo_agg_edge_bwd(_p(indptr), _p(src), _p(edge_w), ctypes.c_int32(edge_w.shape[1]), _p(dy), ctypes.c_int64(D),
                            ctypes.c_int32(D), ctypes.c_int32(n_dst), ctypes.c_int32(n_src), _p(dx), ctypes.c_int64(D))
    return dx
