"""The allocation-free SpMM entry point, `cagnet_spmm_csr_f32_noalloc`, called through the C ABI.

Who needs it: a host that cannot get device memory at the moment of the call.  Typical cases are a serving
process in which some other allocator was given the whole GPU at start-up, so `cudaMalloc` just fails, and a
latency-critical loop that cannot afford the device-wide synchronisation `cudaMalloc` / `cudaFree` imply.
The ordinary entry point needs a caller-allocated plan buffer; this one keeps the plan in a fixed device
array inside the library and so allocates nothing.

What is checked: its output against the ordinary entry point's on the same inputs and against an fp64 product
from the CPU oracle's definition, within the tolerance the other kernel tests use (1e-4 of the largest
magnitude), for two calls in a row.  The second call uses a different matrix with fewer hub rows, so a list left
over from the first call would show up as wrong rows; and no device memory may have been taken between the
moment before it and the moment after it (the first call is the warm-up that loads the module).
This file is named to be collected last and does not depend on anything the other tests leave behind.
"""
import ctypes

import pytest
import torch

from cagnet_b200 import _native, ops, partition as PP

pytestmark = pytest.mark.gpu
REL = 1e-4


def _block(n, m, avg, hubs, seed):
    g = torch.Generator().manual_seed(seed)
    r = torch.randint(0, n, (n * avg,), generator=g)
    c = torch.randint(0, m, (n * avg,), generator=g)
    for h in range(hubs):                                   # rows far beyond the hub-row threshold
        extra = torch.randperm(m, generator=g)[: min(m, 9000)]
        r = torch.cat([r, torch.full_like(extra, (11 * h + 2) % n)])
        c = torch.cat([c, extra])
    blk = PP.coalesce_block(r, c, n, m)
    return PP.Block(blk.rows, blk.cols, torch.randn(blk.vals.numel(), generator=g), n, m)


def _call_noalloc(A, B, C, beta):
    lib = _native.lib()
    rc = lib.cagnet_spmm_csr_f32_noalloc(A.rowptr.data_ptr(), A.col.data_ptr(), A.val.data_ptr(), A.n, A.m, A.nnz,
                                         B.data_ptr(), B.stride(0), C.data_ptr(), C.stride(0), B.size(1),
                                         ctypes.c_float(beta), torch.cuda.current_stream().cuda_stream)
    _native.check(rc, "spmm_noalloc")


def _rel_err(got, want):
    return float((got.double() - want.double()).abs().max() / max(float(want.double().abs().max()), 1e-30))


def test_noalloc_matches_the_planned_entry_point_twice_in_a_row():
    cases = [(_block(3000, 12000, 12, hubs=6, seed=1), 41, 0.0),
             (_block(1500, 10000, 5, hubs=1, seed=2), 602, 1.0)]
    for call, (blk, f, beta) in enumerate(cases):
        A = ops.CsrBlock.from_coo(blk.rows, blk.cols, blk.vals, blk.n_rows, blk.n_cols)      # builds its own plan
        assert A.long_rows() >= 1
        g = torch.Generator().manual_seed(f)
        Bh = torch.randn(blk.n_cols, f, generator=g)
        B = ops.to_padded(Bh.cuda())
        C0 = torch.randn(blk.n_rows, f, generator=g).cuda()
        want = ops.to_padded(C0)
        ops.spmm(A, B, want, beta)                                                            # existing entry point
        got = ops.to_padded(C0)
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        _call_noalloc(A, B, got, beta)
        torch.cuda.synchronize()
        if call > 0:                          # from the second call on the entry point takes no device memory at all
            assert torch.cuda.mem_get_info()[0] == free_before
        assert _rel_err(got, want) <= REL
        dense64 = torch.sparse_coo_tensor(torch.stack([blk.rows, blk.cols]), blk.vals.double(), (blk.n_rows, blk.n_cols))
        oracle = torch.sparse.mm(dense64, Bh.double()) + beta * C0.double().cpu()
        assert _rel_err(got.cpu(), oracle) <= REL


def test_noalloc_rejects_sizes_beyond_its_scratch():
    lib = _native.lib()
    limit = lib.cagnet_spmm_noalloc_max_nnz()
    assert limit == 65535 * _native.get_param("spmm_long")
    if limit + 1 < 2 ** 31:
        # the size check comes before any pointer is touched, so dummy non-null pointers are enough
        rc = lib.cagnet_spmm_csr_f32_noalloc(8, 8, 8, 4, 4, limit + 1, 8, 4, 8, 4, 4, ctypes.c_float(0.0), None)
        assert rc == 5
        assert b"exceed the built-in scratch" in lib.cagnet_last_error_string()
