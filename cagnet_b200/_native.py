"""ctypes binding of `libcagnet_b200.so` (the C ABI declared in include/cagnet_b200.h).

There is no fallback: if the library has not been built, or a call fails, this raises.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libcagnet_b200.so")

_vp, _i32, _i64, _f32, _sz, _cp = (ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64, ctypes.c_float,
                                   ctypes.c_size_t, ctypes.c_char_p)

# name -> (restype, argtypes); mirrors include/cagnet_b200.h one to one
PROTOTYPES = {
    "cagnet_version": (_i32, []),
    "cagnet_last_error_string": (_cp, []),
    "cagnet_set_param": (_i32, [_cp, _i32]),
    "cagnet_get_param": (_i32, [_cp]),
    "cagnet_coo2csr_i32": (_i32, [_vp, _i64, _i32, _vp, _vp]),
    "cagnet_check_csr_i32": (_i32, [_vp, _vp, _vp, _i32, _i32, _i64, _vp, _vp]),
    "cagnet_spmm_plan_bytes": (_sz, [_i32, _i64]),
    "cagnet_spmm_plan_i32": (_i32, [_vp, _i32, _i64, _vp, _sz, _vp]),
    "cagnet_spmm_csr_f32": (_i32, [_vp, _vp, _vp, _i32, _i32, _i64, _vp, _i64, _vp, _i64, _i32, _f32, _vp, _vp]),
    "cagnet_spmm_noalloc_max_nnz": (_i64, []),
    "cagnet_spmm_csr_f32_noalloc": (_i32, [_vp, _vp, _vp, _i32, _i32, _i64, _vp, _i64, _vp, _i64, _i32, _f32, _vp]),
    "cagnet_core_gemm_workspace_bytes": (_sz, [_i32, _i32, _i32]),
    "cagnet_core_gemm_f32": (_i32, [_vp, _i64, _vp, _i32, _vp, _i32, _vp, _i64, _vp, _i64, _i32, _vp, _sz, _vp]),
    "cagnet_core_gemm_tc_available": (_i32, []),
    "cagnet_core_gemm_tc_workspace_bytes": (_sz, [_i32, _i32, _i32]),
    "cagnet_split_tf32_f32": (_i32, [_vp, _i64, _vp, _vp, _vp]),
    "cagnet_gather_split_rows_f32": (_i32, [_vp, _i64, _vp, _i32, _i32, _vp, _i64, _vp]),
    "cagnet_core_gemm_tc_f32": (_i32, [_vp, _vp, _i64, _i32, _i32, _vp, _i64, _vp, _i32, _vp, _sz, _vp]),
    "cagnet_add_rows3_f32": (_i32, [_vp, _i64, _vp, _i32, _i32, _vp, _i64, _vp]),
    "cagnet_core_gemm_int_available": (_i32, []),
    "cagnet_core_gemm_int_workspace_bytes": (_sz, [_i32, _i32, _i32]),
    "cagnet_gather_scale_split3_bf16": (_i32, [_vp, _i64, _vp, _vp, _i32, _i32, _vp, _i64, _vp]),
    "cagnet_core_gemm_int_bf16": (_i32, [_vp, _i64, _i32, _i32, _vp, _i64, _vp, _i32, _vp, _sz, _vp]),
    "cagnet_add_rows_scaled3_f32": (_i32, [_vp, _i64, _vp, _vp, _i32, _i32, _vp, _i64, _vp]),
    "cagnet_gemm_nn_f32": (_i32, [_vp, _i64, _vp, _i64, _i32, _vp, _i64, _i64, _i32, _i32, _i32, _vp, _i64, _vp]),
    "cagnet_gemm_tn_workspace_bytes": (_sz, [_i64, _i32, _i32]),
    "cagnet_gemm_tn_f32": (_i32, [_vp, _i64, _vp, _i64, _vp, _i64, _i64, _i32, _i32, _f32, _vp, _sz, _vp]),
    "cagnet_row_reduce_f32": (_i32, [_vp, _i64, _i64, _i32, _i32, _vp, _vp, _vp]),
    "cagnet_log_softmax_apply_f32": (_i32, [_vp, _i64, _vp, _vp, _vp, _i64, _i64, _i32, _vp]),
    "cagnet_log_softmax_bwd_apply_f32": (_i32, [_vp, _i64, _vp, _i64, _vp, _vp, _i64, _i64, _i32, _vp]),
    "cagnet_relu_fwd_f32": (_i32, [_vp, _i64, _vp, _i64, _i64, _i32, _vp]),
    "cagnet_relu_bwd_f32": (_i32, [_vp, _i64, _vp, _i64, _vp, _i64, _i64, _i32, _vp]),
    "cagnet_log_softmax_fwd_f32": (_i32, [_vp, _i64, _vp, _i64, _i64, _i32, _vp]),
    "cagnet_log_softmax_bwd_f32": (_i32, [_vp, _i64, _vp, _i64, _vp, _i64, _i64, _i32, _vp]),
    "cagnet_nll_workspace_bytes": (_sz, [_i64]),
    "cagnet_nll_masked_f32": (_i32, [_vp, _i64, _vp, _vp, _i64, _i32, _i32, _i32, _f32, _f32, _vp, _vp, _i64, _vp,
                                     _sz, _vp]),
}

_lib = None


def lib():
    """The loaded library; raises RuntimeError with build instructions if it is missing."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                "cagnet_b200: native library %s is missing; build it with `python -m cagnet_b200.build` "
                "(there is no CPU or PyTorch fallback)" % LIB_PATH)
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def check(status, what=""):
    if status != 0:
        msg = lib().cagnet_last_error_string()
        raise RuntimeError("cagnet_b200 %s failed with status %d: %s" % (what, status, msg.decode() if msg else "?"))


def set_param(name, value):
    check(lib().cagnet_set_param(name.encode(), int(value)), "set_param")


def get_param(name):
    return lib().cagnet_get_param(name.encode())
