"""CPU-side checks of the drop-in boundary: the library loads, exports what the header declares, and the
product path refuses CPU tensors instead of falling back."""
import os
import re

import pytest
import torch

from cagnet_b200 import _native, ops

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "cagnet_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(cagnet_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _native.lib()
    names = _declared()
    assert len(names) >= 18
    for name in names:
        assert hasattr(lib, name), name
    assert sorted(_native.PROTOTYPES) == names          # the ctypes table mirrors the header one to one
    assert lib.cagnet_version() >= 100


def test_host_side_queries_need_no_gpu():
    lib = _native.lib()
    assert lib.cagnet_spmm_plan_bytes(1000, 50000) >= 32
    assert lib.cagnet_gemm_tn_workspace_bytes(100000, 602, 16) >= 602 * 16 * 4
    assert lib.cagnet_nll_workspace_bytes(10) > 0
    assert _native.get_param("spmm_long") >= 256
    with pytest.raises(RuntimeError, match="unknown parameter"):
        _native.set_param("no_such_knob", 1)
    with pytest.raises(RuntimeError, match="spmm_long"):
        _native.set_param("spmm_long", 3)


def test_argument_errors_are_status_codes_not_crashes():
    lib = _native.lib()
    assert lib.cagnet_spmm_csr_f32(None, None, None, -1, 1, 0, None, 1, None, 1, 1, 0.0, None, None) == 1
    assert b"negative" in lib.cagnet_last_error_string()
    assert lib.cagnet_coo2csr_i32(None, 5, 3, None, None) == 1
    assert lib.cagnet_check_csr_i32(None, None, None, 1, 1, 0, None, None) == 1
    assert lib.cagnet_gemm_nn_f32(None, 1, None, 1, 0, None, 1, 4, 4, 4, 0, None, 0, None) == 1
    # fused log-softmax wider than one tile is refused
    assert lib.cagnet_gemm_nn_f32(1, 100, 1, 100, 0, 1, 100, 4, 4, 100, 2, None, 0, None) == 1
    # nnz beyond int32
    assert lib.cagnet_coo2csr_i32(1, 2 ** 31, 3, 1, None) == 3


def test_dense_core_entry_points_validate_before_launching():
    lib = _native.lib()
    p = 0x7f0000000000                      # never dereferenced: every call below fails its argument checks
    assert lib.cagnet_core_gemm_workspace_bytes(0, 10, 10) == 0
    assert lib.cagnet_core_gemm_workspace_bytes(4096, 13312, 602) >= 4096 * 604 * 4
    assert lib.cagnet_core_gemm_f32(p, 8, p, -1, p, 8, p, 8, p, 8, 8, None, 0, None) == 1
    assert lib.cagnet_core_gemm_f32(p, 4, p, 8, p, 8, p, 8, p, 8, 8, None, 0, None) == 1        # ld_core < K
    assert lib.cagnet_core_gemm_f32(p, 8, p, 8, p, 8, p, 7, p, 8, 7, None, 0, None) == 2        # B rows unaligned
    assert lib.cagnet_core_gemm_f32(p, 13312, p, 4096, p, 13312, p, 608, p, 608, 602, None, 0, None) == 5   # no scratch
    assert lib.cagnet_core_gemm_f32(p, 8, p, 0, p, 8, p, 8, p, 8, 8, None, 0, None) == 0        # nothing to do
    assert lib.cagnet_split_tf32_f32(None, 0, None, None, None) == 0
    assert lib.cagnet_split_tf32_f32(None, 5, None, None, None) == 1
    assert lib.cagnet_gather_split_rows_f32(p, 6, p, 4, 6, p, 8, None) == 2                     # ldb not a multiple of 4
    assert lib.cagnet_gather_split_rows_f32(p, 8, p, 4, 6, p, 4, None) == 2                     # half < f rounded up
    assert lib.cagnet_add_rows3_f32(p, 6, p, 4, 6, p, 8, None) == 2
    assert lib.cagnet_add_rows3_f32(p, 8, p, 4, 6, p, 4, None) == 2                             # ldc < f
    assert lib.cagnet_core_gemm_tc_available() in (0, 1)
    if lib.cagnet_core_gemm_tc_available():
        assert lib.cagnet_core_gemm_tc_workspace_bytes(4096, 4096, 602) >= 16
        assert lib.cagnet_core_gemm_tc_f32(p, p, 8, 4, 16, p, 8, p, 8, None, 0, None) == 1      # ld_core < K
        assert lib.cagnet_core_gemm_tc_f32(p, p, 18, 4, 16, p, 8, p, 8, None, 0, None) == 2     # ld_core % 4
    else:
        assert lib.cagnet_core_gemm_tc_f32(p, p, 16, 4, 16, p, 8, p, 8, None, 0, None) == 1


def test_cpu_tensors_are_refused():
    blk = ops.CsrBlock(torch.zeros(3, dtype=torch.int32), torch.zeros(0, dtype=torch.int32), torch.zeros(0), 2, 2)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        ops.spmm(blk, torch.zeros(2, 4), torch.zeros(2, 4))
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        ops.gemm_nn(torch.zeros(4, 4), torch.zeros(4, 4))
    with pytest.raises(RuntimeError, match="int32 CUDA"):
        ops.coo2csr(torch.zeros(3, dtype=torch.int32), 4)


def test_padded_layout_helpers():
    assert [ops.pad_ld(f) for f in (1, 16, 41, 64, 65, 300, 602)] == [4, 16, 44, 64, 96, 320, 608]
    v = ops.zeros_padded(5, 41, "cpu")
    assert v.shape == (5, 41) and v.stride() == (44, 1)
    assert ops.base_buffer(v).shape == (5, 44)
    c = torch.zeros(5, 16)
    assert ops.base_buffer(c) is c
