"""CPU checks of the drop-in boundary: the C-ABI library loads without a GPU, exports every symbol the
header declares, and the Python ops reject what the reference's CHECK_INPUT rejects."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "fastgl_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fgl_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from fastgl import _capi
    handle = ctypes.CDLL(_capi.LIB_PATH)
    names = declared_symbols()
    assert len(names) >= 15
    for name in names:
        assert hasattr(handle, name), name
    assert sorted(_capi.EXPORTS) == names


def test_abi_version_struct_layout_and_status_strings():
    from fastgl import _capi
    lib = _capi.lib()
    assert lib.fgl_abi_version() == _capi.ABI_VERSION
    assert lib.fgl_sizeof_fused_args() == ctypes.sizeof(_capi.FusedArgs)
    assert _capi.status_str(0) == "ok"
    assert "probe" in _capi.status_str(5)


def test_capacity_helper_matches_the_hop_sizes():
    import fastgl
    # batch 1024, hops 5 / 10 / 15: 1024 -> 6144 -> 67584 -> 1081344 nodes at most
    assert fastgl.fused_capacity(2_450_000, 1024, [5, 10, 15]) == [1024, 6144, 67584, 1081344]
    # the node count caps the frontier
    assert fastgl.fused_capacity(50_000, 1024, [5, 10, 15]) == [1024, 6144, 50000, 50000]
    with pytest.raises(RuntimeError):
        fastgl.fused_capacity(1000, 10, [0])


def test_invalid_arguments_return_status_without_touching_a_device():
    from fastgl import _capi
    lib = _capi.lib()
    assert lib.fgl_sample(None, None, 0, None, ctypes.c_int64(0), None, 0, 0, 0, ctypes.c_uint64(0), ctypes.c_uint64(0),
                          None, None, None, None, None) == 1
    assert lib.fgl_agg_fwd(None, 9, None, None, None, None, None, ctypes.c_int64(0), None, ctypes.c_int64(1),
                           ctypes.c_int64(4), 4, 1, 0, None, ctypes.c_int64(4), None, None) == 1
    assert lib.fgl_exclusive_sum_noalloc_status(None, None) == 1
    assert lib.fgl_selftest_barrier_timeout(None, 1, ctypes.c_int64(10), None) == 1
    assert lib.fgl_ws_destroy(None) == 0
    # the entry points of the error-compensated products, the access probe and the launch timer
    one = (ctypes.c_void_p * 1)(1)
    ld = (ctypes.c_int64 * 1)(4)
    part = (ctypes.c_int32 * 1)(0)
    i64 = ctypes.c_int64
    assert lib.fgl_split_tf32(None, i64(-1), i64(4), i64(4), 1, one, ld, part, None) == 1          # negative row count
    assert lib.fgl_split_tf32(None, i64(2), i64(8), i64(4), 1, one, ld, part, None) == 1           # ldx < cols
    assert lib.fgl_split_tf32(None, i64(2), i64(4), i64(4), 9, one, ld, part, None) == 1           # too many destinations
    assert lib.fgl_split_tf32(None, i64(0), i64(4), i64(4), 1, one, ld, part, None) == 0           # nothing to do
    assert lib.fgl_relu_dropout_bwd_split(None, i64(4), None, i64(4), i64(2), 4, ctypes.c_float(0.0), None, 0, None, i64(12),
                                          i64(4), None) == 1                                        # no destination
    assert lib.fgl_fold_blocks(None, 0, 2, 2, 4, 4, 4, i64(8), i64(64), None, i64(4), None) == 1     # no slabs
    assert lib.fgl_fold_blocks(None, 1, 2, 2, 4, 4, 2, i64(8), i64(64), None, i64(4), None) == 1     # blocks overlap
    assert lib.fgl_fold_blocks(None, 1, 2, 2, 0, 4, 4, i64(8), i64(0), None, i64(4), None) == 0      # empty result
    n = i64(0)
    assert lib.fgl_probe_access_pattern(None, i64(16), None, i64(0), 1, None, ctypes.byref(n), None) == 1
    assert lib.fgl_ws_time_next_launch(None, None, None) == 1


def test_ops_reject_cpu_and_non_contiguous_tensors():
    import fastgl
    idx = torch.zeros(4, dtype=torch.int32)
    feat = torch.zeros((4, 4))
    with pytest.raises(RuntimeError, match="CUDA"):
        fastgl.cal_deg(idx, 4)
    with pytest.raises(RuntimeError, match="CUDA"):
        fastgl.sample_node(idx, idx, idx, idx, 4, 2)
    with pytest.raises(RuntimeError, match="CUDA"):
        fastgl.transfer_edge_id(idx, idx, idx, 4, 8, 4, 4)
    with pytest.raises(RuntimeError, match="CUDA"):
        fastgl.forwaed_gin(idx, idx, feat, feat, 2, 4)
    with pytest.raises(RuntimeError, match="CUDA"):
        fastgl.forward_gcn(idx, idx, idx, idx, feat, feat, 2, 4)


def test_reference_op_names_are_exposed():
    import fastgl
    for name in ("sample_node", "transfer_edge_id", "cal_deg", "exclusive_sum", "forward_gcn", "backward_gcn",
                 "forwaed_gin", "backward_gin", "forward_gat", "backward_gat"):
        assert callable(getattr(fastgl, name))
