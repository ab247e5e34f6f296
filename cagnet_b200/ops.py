"""Torch-facing wrappers of the C ABI: device tensors in, kernels launched on the current stream.

Mirrors the reference's native operator surface (`sparse_coo_tensor_cpp.spmm_gpu`,
`sparse_coo_tensor_cpp.sparse_coo_tensor_gpu`; sparse-extension/sparse_coo_tensor.cu:43-54, 113-240)
and adds the cached-CSR form the GCN layers use.  PyTorch is the owner of device memory and streams
here; every multiply, activation and loss is a kernel of `libcagnet_b200.so` (torch index kernels are used
once per block, when its dense core is looked for and cut out).  CPU tensors are rejected.
"""
import os

import torch

from . import _native, core_select

EPI_NONE, EPI_RELU, EPI_LOG_SOFTMAX, EPI_RELU_MASK, EPI_ACCUMULATE = 0, 1, 2, 3, 4
_INT32_MAX = 2 ** 31 - 1

# kernels of the native library launched by this process (every wrapper below adds what it launches)
LAUNCHES = [0]


def launch_count():
    return LAUNCHES[0]


def _stream():
    """Raw handle of torch's current stream on the current device (the direct binding: building a
    torch.cuda.Stream object per launch costs more host time than the launch itself)."""
    return torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice())


class _NoSwitch:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


_NO_SWITCH = _NoSwitch()


def _on(device):
    """Context that makes `device` current for a launch; free when it already is (the common case)."""
    if device.index is None or device.index == torch._C._cuda_getDevice():
        return _NO_SWITCH
    return torch.cuda.device(device)


def pad_ld(f):
    """Leading dimension used for matrices this package allocates: rows start on a 16-byte boundary
    (128-bit loads) and, for wide rows, on a 128-byte cache line."""
    return (f + 3) // 4 * 4 if f <= 64 else (f + 31) // 32 * 32


def _alias(storage_of, offset, shape, stride):
    """A tensor over existing storage that autograd does not treat as a view of anything."""
    out = torch.empty(0, dtype=torch.float32, device=storage_of.device)
    return out.set_(storage_of.untyped_storage(), offset, shape, stride)


def empty_padded(n, f, device):
    """n x f fp32 matrix with strides (pad_ld(f), 1) over a buffer of n * ld elements; pad columns unspecified."""
    ld = pad_ld(f)
    flat = torch.empty(max(n * ld, 1), dtype=torch.float32, device=device)
    return _alias(flat, 0, (n, f), (ld, 1))


def zeros_padded(n, f, device):
    ld = pad_ld(f)
    flat = torch.zeros(max(n * ld, 1), dtype=torch.float32, device=device)
    return _alias(flat, 0, (n, f), (ld, 1))


def to_padded(x):
    """Copy of x (n x f) in the padded layout (pad columns zero)."""
    out = zeros_padded(x.size(0), x.size(1), x.device)
    out.copy_(x)
    return out


def base_buffer(x):
    """The contiguous n x ld buffer behind a padded matrix (what a collective must move, pad columns included),
    or x itself when it is already contiguous."""
    if x.is_contiguous():
        return x
    if x.dim() == 2 and x.stride(1) == 1 and x.stride(0) >= x.size(1):
        n, ld = x.size(0), x.stride(0)
        need = (x.storage_offset() + n * ld) * x.element_size()
        if x.untyped_storage().nbytes() >= need:
            return _alias(x, x.storage_offset(), (n, ld), (ld, 1))
    raise RuntimeError("cagnet_b200: tensor is neither contiguous nor a padded row-major matrix")


def is_padded(x):
    """True if x is a device fp32 matrix already in the layout `empty_padded` produces."""
    if not (x.is_cuda and x.dtype == torch.float32 and x.dim() == 2):
        return False
    if x.size(0) > 1 and x.stride(0) != pad_ld(x.size(1)):
        return False
    if x.size(1) > 1 and x.stride(1) != 1:
        return False
    if x.storage_offset() % pad_ld(x.size(1)) != 0:      # a column slice of a wider matrix is not a padded matrix
        return False
    try:
        base_buffer(x)
    except RuntimeError:
        return False
    return True


def _ld(t, name):
    if not t.is_cuda:
        raise RuntimeError("cagnet_b200: %s must be a CUDA tensor (there is no CPU path)" % name)
    if t.dtype != torch.float32 or t.dim() != 2:
        raise RuntimeError("cagnet_b200: %s must be a 2-D float32 tensor" % name)
    rows, cols = t.shape
    if cols > 1 and t.stride(1) != 1:
        raise RuntimeError("cagnet_b200: %s must be row-major (unit column stride)" % name)
    if rows > 1:
        if t.stride(0) < cols:
            raise RuntimeError("cagnet_b200: %s has overlapping rows" % name)
        return t.stride(0)
    return max(cols, 1)


def _row_major(t):
    return t.dim() == 2 and (t.size(1) <= 1 or t.stride(1) == 1) and (t.size(0) <= 1 or t.stride(0) >= t.size(1))


# Dense-core extraction (see CsrBlock.extract_core).  "density": a rectangle of hub rows x hub columns is worth
# multiplying densely when more than this share of its cells are nonzeros (gathering one 2.4 KB row of B per
# nonzero costs about five dense cells at width 602); "step": side lengths tried are multiples of this;
# "max_side" / "max_bytes": limits of the rectangle; "min_share": the rectangle must save at least this share of
# the block's nonzero-gathers to be cut out (the gathers a core removes are the cheap ones, rows of B that live in
# L2: on edge-factor-16 R-MAT graphs, whose cost is the DRAM-bound rest, cores worth 4-5 % measured -2 % .. +10 %); "min_width": products narrower than this keep using the full CSR
# block (they are bound per nonzero, not per byte, and a 128-column dense tile would be mostly padding); "rounds":
# how many rectangles may be cut out one after the other (a second one, 9,216 x 4,096 at 30 % density on the
# benchmark graph, measured no gain: 13.30 ms against 13.13 ms).
# "tensor_cores": multiply the core with the tcgen05 kernel when the library was built with it (fp32 accuracy
# through the hi/lo TF32 split, "3xTF32": 172 TFLOP/s fp32-equivalent against 40 for the fp32-FMA kernel); a dense
# cell then costs a twelfth of a gathered nonzero and "density_tc" is the bar instead of "density".
# "min_row_nnz": blocks with fewer nonzeros per row on average are left all-sparse whatever their hub rectangle looks
# like: their multiply waits on the latency of scattered DRAM gathers, and taking the cheap, cache-resident hub
# entries out of it saves nothing (R-MAT with 31 nonzeros per row, 4 M vertices, integer core worth 16 % of the
# nonzeros: width 602 34.6 -> 36.2 ms, width 256 13.8 -> 14.4 ms).
# "integer": a block that carries its normalisation factors (partition.Block.row_scale / col_scale) keeps its core
# as the bf16 matrix of edge multiplicities between the two diagonals and multiplies it with three bf16 products
# (csrc/core_gemm_int.cu): a quarter of the memory and a third of the tensor time of the 3xTF32 form, so the bar
# is "density_int", the side limit "max_side_int", and products down to "min_width_int" columns use it.
CORE = {"enabled": os.environ.get("CAGNET_DENSE_CORE", "1") != "0", "density": 0.2, "density_tc": 0.09, "step": 1024,
        "max_side": 16384, "max_bytes": 2 << 30, "min_share": 0.1, "min_width": 128, "rounds": 1,
        "tensor_cores": os.environ.get("CAGNET_CORE_TENSOR", "1") != "0",
        "integer": os.environ.get("CAGNET_CORE_INTEGER", "1") != "0", "density_int": 0.02, "max_side_int": 32768,
        "min_width_int": 128, "min_row_nnz": 64}


def core_on_tensor_cores():
    return bool(CORE["tensor_cores"]) and _native.lib().cagnet_core_gemm_tc_available() == 1


def integer_core_available():
    return bool(CORE["tensor_cores"]) and bool(CORE["integer"]) and _native.lib().cagnet_core_gemm_int_available() == 1


def configure_core(**kw):
    """Change dense-core settings for blocks planned from now on; returns the previous settings."""
    old = dict(CORE)
    for k, v in kw.items():
        if k not in CORE:
            raise KeyError(k)
        CORE[k] = v
    return old


# ------------------------------------------------------------------------------------------ sparse
def coo2csr(rows, n):
    """rowptr[i] = #{e : rows[e] < i} for sorted int32 row indices on the device (int32, n + 1 entries)."""
    if not rows.is_cuda or rows.dtype != torch.int32 or rows.dim() != 1:
        raise RuntimeError("cagnet_b200: coo2csr needs a 1-D int32 CUDA tensor")
    rows = rows.contiguous()
    rowptr = torch.empty(n + 1, dtype=torch.int32, device=rows.device)
    with _on(rows.device):
        _native.check(_native.lib().cagnet_coo2csr_i32(rows.data_ptr(), rows.numel(), n, rowptr.data_ptr(), _stream()),
                      "coo2csr")
    LAUNCHES[0] += 1
    return rowptr


class CsrBlock:
    """A static n x m sparse block on the device: int32 CSR + fp32 values + the SpMM plan (list of hub rows).

    Built once per adjacency block at partition time; the reference instead rebuilds the CSR offsets
    inside every `spmm_gpu` call (sparse_coo_tensor.cu:136-142)."""

    def __init__(self, rowptr, col, val, n, m, plan=None):
        self.rowptr, self.col, self.val, self.n, self.m, self.plan = rowptr, col, val, int(n), int(m), plan
        self.nnz = int(val.numel())
        self.core = self.rest = None      # dense hub-by-hub rectangle and the CSR block of everything else
        self.core_split = None            # the rectangle as TF32 hi + lo parts (tensor-core multiply)
        self.core_int = None              # (bf16 multiplicities, rows, cols, row factors, column factors)
        self.row_scale = self.col_scale = None    # the diagonals a normalised block was scaled with, if known

    @staticmethod
    def from_coo(rows, cols, vals, n, m, validate=True, plan=True, row_scale=None, col_scale=None):
        """rows/cols: integer tensors sorted by row (a coalesced COO), vals fp32; any device (moved to CUDA).
        row_scale / col_scale: the diagonals of a normalised block (see partition.Block), optional."""
        if n > _INT32_MAX or m > _INT32_MAX or vals.numel() > _INT32_MAX:
            raise RuntimeError("cagnet_b200: block does not fit 32-bit indices")
        dev = vals.device if vals.is_cuda else torch.device("cuda", torch.cuda.current_device())
        rows32 = rows.to(device=dev, dtype=torch.int32).contiguous()
        col32 = cols.to(device=dev, dtype=torch.int32).contiguous()
        val = vals.to(device=dev, dtype=torch.float32).contiguous()
        rowptr = coo2csr(rows32, n)
        blk = CsrBlock(rowptr, col32, val, n, m)
        if row_scale is not None and col_scale is not None:
            blk.row_scale = row_scale.to(device=dev, dtype=torch.float32).contiguous()
            blk.col_scale = col_scale.to(device=dev, dtype=torch.float32).contiguous()
        if validate:
            blk.validate(rows32)
        if plan:
            blk.build_plan()
        return blk

    def validate(self, rows=None):
        """Device-side check of the block (and of the sorted COO row indices it came from); one readback."""
        status = torch.zeros(1, dtype=torch.int32, device=self.val.device)
        with _on(self.val.device):
            _native.check(_native.lib().cagnet_check_csr_i32(self.rowptr.data_ptr(), self.col.data_ptr(),
                                                             None if rows is None else rows.data_ptr(), self.n, self.m,
                                                             self.nnz, status.data_ptr(), _stream()), "check_csr")
        LAUNCHES[0] += 1
        code = int(status.item())
        if code:
            reason = {1: "rowptr[0] != 0", 2: "rowptr[n] != nnz (row index out of range or unsorted)",
                      3: "row indices not sorted", 4: "column index out of range",
                      5: "row index out of range"}.get(code, "?")
            raise RuntimeError("cagnet_b200: malformed sparse block: " + reason)

    def build_plan(self, core=True):
        """Hub-row list for the SpMM kernels and, with `core`, the dense-core split for wide products."""
        nbytes = _native.lib().cagnet_spmm_plan_bytes(self.n, self.nnz)
        self.plan = torch.empty((nbytes + 15) // 16 * 16, dtype=torch.uint8, device=self.val.device)
        with _on(self.val.device):
            _native.check(_native.lib().cagnet_spmm_plan_i32(self.rowptr.data_ptr(), self.n, self.nnz,
                                                             self.plan.data_ptr(), self.plan.numel(), _stream()),
                          "spmm_plan")
        LAUNCHES[0] += 5      # header + four length-class passes
        if core:
            self.extract_core()

    def extract_core(self, depth=0):
        """Cut the dense core out of a power-law block.

        Rows and columns are ranked by degree; among the rectangles (top r rows) x (top c columns), r and c
        multiples of CORE["step"], the one with the largest `nonzeros inside - density * cells` is taken if that
        figure is worth it.  Its entries become a dense r x c matrix -- fp32 values (`self.core`, with the row and
        column lists; multiplied by the 3xTF32 or the fp32-FMA kernel), or, when the block carries its normalisation
        factors and its values factor exactly, the bf16 matrix of edge multiplicities with the two factor vectors
        (`self.core_int`; three bf16 tensor-core products) -- and all other entries form `self.rest`, a CSR block
        with its own hub-row plan.  The full block stays as it is for narrow products.  Blocks with fewer than
        CORE["min_row_nnz"] nonzeros per row on average are left alone.  `rest` is searched again
        (the region is L-shaped in a symmetric matrix: hub rows x many columns, then many rows x hub columns), up
        to CORE["rounds"] rectangles.  Runs once per block, with torch index kernels on the block's device; the
        choice depends only on the block (ties broken by index)."""
        cfg = CORE
        if not cfg["enabled"] or self.nnz < cfg["min_row_nnz"] * self.n:
            return
        integer = self.row_scale is not None and integer_core_available()
        if integer:
            bar, side, cell = cfg["density_int"], cfg["max_side_int"], 2
        else:
            bar, side, cell = (cfg["density_tc"] if core_on_tensor_cores() else cfg["density"]), cfg["max_side"], 4
        choice = core_select.choose_core(self.rowptr, self.col, self.n, self.m, bar, cfg["step"], side,
                                         cfg["max_bytes"], cfg["min_share"], cell)
        if choice is None:
            return
        dense, rest_rowptr, rest_col, rest_val = core_select.split_core(self.col, self.val, self.n, choice)
        core_rows, core_cols = choice.rows.int().contiguous(), choice.cols.int().contiguous()
        if integer:
            rs, cs = self.row_scale[choice.rows].contiguous(), self.col_scale[choice.cols].contiguous()
            cnt = core_select.integer_core(dense, rs, cs)
            if cnt is None:
                # the values do not factor (scales of another block, weighted edges): choose again under the fp32
                # rules, which allow less
                del dense, rest_rowptr, rest_col, rest_val
                saved, self.row_scale = self.row_scale, None
                try:
                    return self.extract_core(depth)
                finally:
                    self.row_scale = saved
            self.core_int = (cnt.to(torch.bfloat16), core_rows, core_cols, rs, cs)
            del cnt
            dense = None
        rest = CsrBlock(rest_rowptr, rest_col, rest_val, self.n, self.m)
        rest.row_scale, rest.col_scale = self.row_scale, self.col_scale
        rest.build_plan(core=False)
        if depth + 1 < int(cfg["rounds"]):
            rest.extract_core(depth + 1)
        self.rest = rest
        self.core = (dense, core_rows, core_cols)
        self.core_split = None
        if dense is not None and core_on_tensor_cores() and dense.stride(0) % 4 == 0:
            hi, lo = torch.empty_like(dense), torch.empty_like(dense)
            with _on(dense.device):
                _native.check(_native.lib().cagnet_split_tf32_f32(dense.data_ptr(), dense.numel(), hi.data_ptr(),
                                                                  lo.data_ptr(), _stream()), "split_tf32")
            LAUNCHES[0] += 1
            self.core_split = (hi, lo)

    def core_shape(self):
        """(rows, columns) of the dense core, or None."""
        if self.core is None:
            return None
        m = self.core_int[0] if self.core_int is not None else self.core[0]
        return int(m.size(0)), int(m.size(1))

    def core_kind(self):
        """How the dense core is multiplied: "bf16-integer", "3xtf32", "fp32-fma", or None without a core."""
        if self.core is None:
            return None
        if self.core_int is not None:
            return "bf16-integer"
        return "3xtf32" if (self.core_split is not None and CORE["tensor_cores"]) else "fp32-fma"

    def long_rows(self):
        """Number of rows the plan routes to the block-per-row kernel (synchronises)."""
        return 0 if self.plan is None else int(self.plan[4:8].view(torch.int32).item())

    def bytes_alg(self, f, beta):
        """Algorithmic HBM bytes of one multiply by an m x f matrix: offsets + (col, val) streams + B read once
        + C written (and read when accumulating)."""
        return 4 * (self.n + 1) + 8 * self.nnz + 4 * self.m * f + 4 * self.n * f * (1 + int(beta != 0))


def spmm(block, B, C, beta=1.0):
    """C = beta * C + block @ B in place (beta 0 or 1)."""
    ldb, ldc = _ld(B, "B"), _ld(C, "C")
    if B.size(0) != block.m or C.size(0) != block.n or B.size(1) != C.size(1):
        raise RuntimeError("cagnet_b200: spmm shape mismatch: A %dx%d, B %s, C %s"
                           % (block.n, block.m, tuple(B.shape), tuple(C.shape)))
    if B.device != block.val.device or C.device != block.val.device:
        raise RuntimeError("cagnet_b200: spmm operands on different devices")
    f = B.size(1)
    min_width = CORE["min_width_int"] if block.core_int is not None else CORE["min_width"]
    use_core = block.core is not None and f >= min_width and ldb % 4 == 0 and B.data_ptr() % 16 == 0
    cores, src = [], block
    while use_core and src.core is not None:
        cores.append(src)
        src = src.rest
    with _on(C.device):
        _native.check(_native.lib().cagnet_spmm_csr_f32(
            src.rowptr.data_ptr(), src.col.data_ptr(), src.val.data_ptr(), src.n, src.m, src.nnz,
            B.data_ptr(), ldb, C.data_ptr(), ldc, f, float(beta),
            None if src.plan is None else src.plan.data_ptr(), _stream()), "spmm")
        LAUNCHES[0] += 1 if src.plan is None else 2
        for owner in cores:
            if owner.core_int is not None:
                _core_multiply_int(owner.core_int, B, ldb, C, ldc, f)
            else:
                dense, core_rows, core_cols = owner.core
                _core_multiply(dense, core_rows, core_cols, owner.core_split, B, ldb, C, ldc, f)
    return C


def _core_multiply_int(core_int, B, ldb, C, ldc, f):
    """C[rows] += diag(rs) . (Cnt . (diag(cs) . B[cols])) with Cnt the bf16 multiplicity matrix: the scaled rows of
    B gathered and cut into three bf16 terms, one tensor-core multiply per k chunk against all three, the sum
    scaled and added into C's hub rows (current stream, device already current)."""
    L = _native.lib()
    cnt, core_rows, core_cols, rs, cs = core_int
    r, k = cnt.size(0), cnt.size(1)
    half = (f + 7) // 8 * 8
    Ys = torch.empty(k * 3 * half, dtype=torch.bfloat16, device=C.device)
    D = torch.empty(r * 3 * half, dtype=torch.float32, device=C.device)
    _native.check(L.cagnet_gather_scale_split3_bf16(B.data_ptr(), ldb, core_cols.data_ptr(), cs.data_ptr(), k, f,
                                                    Ys.data_ptr(), half, _stream()), "gather_scale_split3")
    nbytes = L.cagnet_core_gemm_int_workspace_bytes(r, k, f)
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=C.device)
    _native.check(L.cagnet_core_gemm_int_bf16(cnt.data_ptr(), cnt.stride(0), r, k, Ys.data_ptr(), half, D.data_ptr(), f,
                                              ws.data_ptr(), ws.numel(), _stream()), "core_gemm_int")
    _native.check(L.cagnet_add_rows_scaled3_f32(D.data_ptr(), half, core_rows.data_ptr(), rs.data_ptr(), r, f,
                                                C.data_ptr(), ldc, _stream()), "add_rows_scaled3")
    chunk = _native.get_param("core_chunk_int")
    LAUNCHES[0] += 2 + (k + chunk - 1) // chunk


def _core_multiply(dense, core_rows, core_cols, split, B, ldb, C, ldc, f):
    """C[core_rows] += dense @ B[core_cols] on the current stream (device already current)."""
    L = _native.lib()
    r, k = dense.size(0), dense.size(1)
    if split is not None and CORE["tensor_cores"]:
        # tensor-core path (3xTF32): B's hub rows gathered and split into [hi | lo] (TMA cannot follow an index
        # list), the three partial products into a scratch matrix, their sum added into C's hub rows
        hi, lo = split
        half = (f + 3) // 4 * 4
        Bs = torch.empty(k * 2 * half, dtype=torch.float32, device=C.device)
        D = torch.empty(r * 3 * half, dtype=torch.float32, device=C.device)
        _native.check(L.cagnet_gather_split_rows_f32(B.data_ptr(), ldb, core_cols.data_ptr(), k, f, Bs.data_ptr(), half,
                                                     _stream()), "gather_split_rows")
        nbytes = L.cagnet_core_gemm_tc_workspace_bytes(r, k, f)
        ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=C.device)
        _native.check(L.cagnet_core_gemm_tc_f32(hi.data_ptr(), lo.data_ptr(), hi.stride(0), r, k, Bs.data_ptr(), half,
                                                D.data_ptr(), f, ws.data_ptr(), ws.numel(), _stream()), "core_gemm_tc")
        _native.check(L.cagnet_add_rows3_f32(D.data_ptr(), half, core_rows.data_ptr(), r, f, C.data_ptr(), ldc,
                                             _stream()), "add_rows3")
        chunk = _native.get_param("core_chunk")
        LAUNCHES[0] += 2 + 2 * ((k + chunk - 1) // chunk)
        return
    nbytes = L.cagnet_core_gemm_workspace_bytes(r, k, f)
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=C.device)
    _native.check(L.cagnet_core_gemm_f32(dense.data_ptr(), dense.stride(0), core_rows.data_ptr(), r,
                                         core_cols.data_ptr(), k, B.data_ptr(), ldb, C.data_ptr(), ldc, f,
                                         ws.data_ptr(), ws.numel(), _stream()), "core_gemm")
    LAUNCHES[0] += 2 if nbytes else 1      # the multiply and the pass that adds up its k slices


SPMM_GPU_VALIDATE = os.environ.get("CAGNET_SPMM_GPU_VALIDATE", "1") != "0"


def spmm_gpu(A_rowindices, A_colindices, A_values, n, m, B, C, validate=None):
    """Drop-in for `sparse_coo_tensor_cpp.spmm_gpu` (sparse_coo_tensor.cu:113-119): C += A.B in place, A given
    as row-sorted COO with int32 indices.  Value semantics only: strides of B and C are left untouched, exactly
    the n x f elements of C change, and the work is queued on the current stream.

    The indices are checked on the device first (sorted rows, rows in [0, n), columns in [0, m)): one 4-byte
    readback, i.e. one stream synchronisation per call where the reference op synchronises the whole device
    (sparse_coo_tensor.cu:231); an out-of-range column would otherwise be an out-of-bounds gather.
    `validate=False` (or CAGNET_SPMM_GPU_VALIDATE=0) skips the check and the synchronisation for callers whose
    indices are known to be good."""
    if A_rowindices.dtype != torch.int32 or A_colindices.dtype != torch.int32:
        raise RuntimeError("cagnet_b200: spmm_gpu expects int32 indices (call .int() as the reference does)")
    if n > _INT32_MAX or m > _INT32_MAX:
        raise RuntimeError("cagnet_b200: spmm_gpu block does not fit 32-bit indices")
    rows32 = A_rowindices.contiguous()
    block = CsrBlock(coo2csr(rows32, n), A_colindices.contiguous(), A_values.float().contiguous(), n, m)
    if SPMM_GPU_VALIDATE if validate is None else validate:
        block.validate(rows32)
    block.build_plan(core=False)      # a per-call block: the core split only pays when it is reused
    Bc = B if _row_major(B) else B.contiguous()
    if _row_major(C):
        spmm(block, Bc, C, 1.0)
    else:  # e.g. the column-major-strided views the reference's own op leaves behind
        tmp = C.contiguous()
        spmm(block, Bc, tmp, 1.0)
        C.copy_(tmp)


def sparse_coo_tensor_gpu(indices, values, size):
    """Drop-in for `sparse_coo_tensor_cpp.sparse_coo_tensor_gpu` (sparse_coo_tensor.cu:43-54): sparse COO
    constructor without index validation (and so without a device synchronisation)."""
    return torch.sparse_coo_tensor(indices, values, tuple(size), check_invariants=False)


# ------------------------------------------------------------------------------------------- dense
def gemm_nn(X, W, trans_w=False, epilogue=EPI_NONE, aux=None, out=None):
    """epilogue(X @ W) (or X @ W.T when trans_w) for tall X and a small W; result in the padded layout."""
    ldx, ldw = _ld(X, "X"), _ld(W, "W")
    K = X.size(1)
    if trans_w:
        N = W.size(0)
        if W.size(1) != K:
            raise RuntimeError("cagnet_b200: gemm_nn shape mismatch %s x %s^T" % (tuple(X.shape), tuple(W.shape)))
    else:
        N = W.size(1)
        if W.size(0) != K:
            raise RuntimeError("cagnet_b200: gemm_nn shape mismatch %s x %s" % (tuple(X.shape), tuple(W.shape)))
    if out is None:
        out = empty_padded(X.size(0), N, X.device)
    ldz = _ld(out, "out")
    aux_ptr, ldaux = (None, 0) if aux is None else (aux.data_ptr(), _ld(aux, "aux"))
    with _on(X.device):
        _native.check(_native.lib().cagnet_gemm_nn_f32(X.data_ptr(), ldx, W.data_ptr(), ldw, int(bool(trans_w)),
                                                       out.data_ptr(), ldz, X.size(0), K, N, int(epilogue), aux_ptr,
                                                       ldaux, _stream()), "gemm_nn")
    LAUNCHES[0] += 1
    return out


def gemm_tn(H, G, out=None, accumulate=False):
    """H.T @ G for tall H (n x K) and G (n x N): K x N, deterministic summation order.  With `out` and
    accumulate=True the product is added to out in place."""
    ldh, ldg = _ld(H, "H"), _ld(G, "G")
    if H.size(0) != G.size(0):
        raise RuntimeError("cagnet_b200: gemm_tn row mismatch")
    n, K, N = H.size(0), H.size(1), G.size(1)
    if out is None:
        if accumulate:
            raise RuntimeError("cagnet_b200: gemm_tn accumulate needs an output matrix")
        out = torch.empty((K, N), dtype=torch.float32, device=H.device)
    elif tuple(out.shape) != (K, N):
        raise RuntimeError("cagnet_b200: gemm_tn output shape mismatch")
    ldo = _ld(out, "out")
    nbytes = _native.lib().cagnet_gemm_tn_workspace_bytes(n, K, N)
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=H.device)
    with _on(H.device):
        _native.check(_native.lib().cagnet_gemm_tn_f32(H.data_ptr(), ldh, G.data_ptr(), ldg, out.data_ptr(), ldo,
                                                       n, K, N, 1.0 if accumulate else 0.0, ws.data_ptr(), ws.numel(),
                                                       _stream()), "gemm_tn")
    LAUNCHES[0] += 2
    return out


ROW_MAX, ROW_SUM, ROW_SUMEXP = 0, 1, 2


def row_reduce(z, mode, ref=None):
    """Per-row max / sum / sum of exp(z - ref) over the columns of z: fp32 vector of n entries."""
    out = torch.empty(z.size(0), dtype=torch.float32, device=z.device)
    with _on(z.device):
        _native.check(_native.lib().cagnet_row_reduce_f32(z.data_ptr(), _ld(z, "z"), z.size(0), z.size(1), int(mode),
                                                          None if ref is None else ref.data_ptr(), out.data_ptr(),
                                                          _stream()), "row_reduce")
    LAUNCHES[0] += 1
    return out


def log_softmax_apply(z, row_max, row_sum):
    out = empty_padded(z.size(0), z.size(1), z.device)
    with _on(z.device):
        _native.check(_native.lib().cagnet_log_softmax_apply_f32(z.data_ptr(), _ld(z, "z"), row_max.data_ptr(),
                                                                 row_sum.data_ptr(), out.data_ptr(), _ld(out, "out"),
                                                                 z.size(0), z.size(1), _stream()), "log_softmax_apply")
    LAUNCHES[0] += 1
    return out


def log_softmax_bwd_apply(logp, g, row_sum_g):
    out = empty_padded(logp.size(0), logp.size(1), logp.device)
    with _on(logp.device):
        _native.check(_native.lib().cagnet_log_softmax_bwd_apply_f32(
            logp.data_ptr(), _ld(logp, "logp"), g.data_ptr(), _ld(g, "g"), row_sum_g.data_ptr(), out.data_ptr(),
            _ld(out, "out"), logp.size(0), logp.size(1), _stream()), "log_softmax_bwd_apply")
    LAUNCHES[0] += 1
    return out


def relu(z):
    out = empty_padded(z.size(0), z.size(1), z.device)
    with _on(z.device):
        _native.check(_native.lib().cagnet_relu_fwd_f32(z.data_ptr(), _ld(z, "z"), out.data_ptr(), _ld(out, "out"),
                                                        z.size(0), z.size(1), _stream()), "relu_fwd")
    LAUNCHES[0] += 1
    return out


def relu_bwd(h, g):
    out = empty_padded(h.size(0), h.size(1), h.device)
    with _on(h.device):
        _native.check(_native.lib().cagnet_relu_bwd_f32(h.data_ptr(), _ld(h, "h"), g.data_ptr(), _ld(g, "g"),
                                                        out.data_ptr(), _ld(out, "out"), h.size(0), h.size(1),
                                                        _stream()), "relu_bwd")
    LAUNCHES[0] += 1
    return out


def log_softmax(z):
    out = empty_padded(z.size(0), z.size(1), z.device)
    with _on(z.device):
        _native.check(_native.lib().cagnet_log_softmax_fwd_f32(z.data_ptr(), _ld(z, "z"), out.data_ptr(),
                                                               _ld(out, "out"), z.size(0), z.size(1), _stream()),
                      "log_softmax_fwd")
    LAUNCHES[0] += 1
    return out


def log_softmax_bwd(logp, g):
    out = empty_padded(logp.size(0), logp.size(1), logp.device)
    with _on(logp.device):
        _native.check(_native.lib().cagnet_log_softmax_bwd_f32(logp.data_ptr(), _ld(logp, "logp"), g.data_ptr(),
                                                               _ld(g, "g"), out.data_ptr(), _ld(out, "out"),
                                                               logp.size(0), logp.size(1), _stream()),
                      "log_softmax_bwd")
    LAUNCHES[0] += 1
    return out


def nll_masked(logp, y, mask, count, cls_lo=0, cls_hi=None, scale=1.0, want_grad=True):
    """(loss, grad): loss = -sum_{mask} logp[i, y_i - cls_lo] / count over rows whose label is in
    [cls_lo, cls_hi); grad = d(scale * loss)/d logp as a dense padded matrix (or None)."""
    n, N = logp.shape
    cls_hi = cls_lo + N if cls_hi is None else cls_hi
    if y.dtype != torch.int64 or not y.is_cuda or mask.dtype not in (torch.bool, torch.uint8) or not mask.is_cuda:
        raise RuntimeError("cagnet_b200: nll_masked needs int64 labels and a bool/uint8 mask on the device")
    y = y.contiguous()
    mask_u8 = mask.contiguous().view(torch.uint8)
    loss = torch.empty((), dtype=torch.float32, device=logp.device)
    grad = empty_padded(n, N, logp.device) if want_grad else None
    nbytes = _native.lib().cagnet_nll_workspace_bytes(n)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=logp.device)
    with _on(logp.device):
        _native.check(_native.lib().cagnet_nll_masked_f32(
            logp.data_ptr(), _ld(logp, "logp"), y.data_ptr(), mask_u8.data_ptr(), n, N, int(cls_lo), int(cls_hi),
            float(count), float(scale), loss.data_ptr(), None if grad is None else grad.data_ptr(),
            0 if grad is None else _ld(grad, "grad"), ws.data_ptr(), ws.numel(), _stream()), "nll_masked")
    LAUNCHES[0] += 2
    return loss, grad
