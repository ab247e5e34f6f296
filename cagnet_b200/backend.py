"""The local-compute interface the distributed schedules are written against.

`CudaBackend` is the product: every method launches kernels of `libcagnet_b200.so` on the current
stream and refuses anything that is not a CUDA tensor.  The schedules take the backend as an argument so
that their communication logic can be exercised over Gloo with CPU tensors by the tests, which pass
their own checker backend; nothing in this package provides a CPU implementation.
"""
import torch

from . import ops

ACT_NONE, ACT_RELU, ACT_LOG_SOFTMAX = "none", "relu", "log_softmax"
_EPI = {ACT_NONE: ops.EPI_NONE, ACT_RELU: ops.EPI_RELU, ACT_LOG_SOFTMAX: ops.EPI_LOG_SOFTMAX}


class CudaBackend:
    name = "cuda"

    def __init__(self, device=None):
        if not torch.cuda.is_available():
            raise RuntimeError("cagnet_b200: no CUDA device; this package has no CPU execution path")
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.spmm_events = None      # when a list: (block, f, beta, start event, stop event) per multiply

    def start_spmm_timing(self):
        """Bracket every following SpMM with CUDA events on the launching stream (for the benchmark's roofline)."""
        self.spmm_events = []

    def stop_spmm_timing(self):
        """Synchronise and return [(n, m, nnz, f, beta, milliseconds)] for the multiplies since start."""
        events, self.spmm_events = self.spmm_events or [], None
        torch.cuda.synchronize(self.device)
        return [(b.n, b.m, b.nnz, f, beta, e0.elapsed_time(e1)) for (b, f, beta, e0, e1) in events]

    # ---- sparse
    def make_block(self, block):
        """partition.Block (COO, any device) -> device CSR with its SpMM plan."""
        return ops.CsrBlock.from_coo(block.rows, block.cols, block.vals, block.n_rows, block.n_cols,
                                     row_scale=getattr(block, "row_scale", None),
                                     col_scale=getattr(block, "col_scale", None))

    def block_shape(self, blk):
        return blk.n, blk.m

    def spmm(self, blk, B, C, beta):
        if self.spmm_events is None:
            return ops.spmm(blk, B, C, beta)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        ops.spmm(blk, B, C, beta)
        e1.record()
        self.spmm_events.append((blk, B.size(1), beta, e0, e1))
        return C

    # ---- storage
    def empty(self, n, f):
        return ops.empty_padded(n, f, self.device)

    def zeros(self, n, f):
        return ops.zeros_padded(n, f, self.device)

    def as_matrix(self, x):
        """Any n x f float tensor -> device matrix in the padded layout (no copy if it already is one)."""
        x = x.detach()
        if ops.is_padded(x):
            return x
        return ops.to_padded(x.to(device=self.device, dtype=torch.float32))

    def wire(self, x):
        """The contiguous buffer a collective moves for matrix x (includes the pad columns)."""
        return ops.base_buffer(x)

    # ---- dense
    def mm(self, X, W, act=ACT_NONE):
        n_out = W.size(1)
        if act == ACT_LOG_SOFTMAX and n_out > 64:
            return ops.log_softmax(ops.gemm_nn(X, W, False, ops.EPI_NONE))
        return ops.gemm_nn(X, W, False, _EPI[act])

    def mm_nt(self, X, W):
        return ops.gemm_nn(X, W, True, ops.EPI_NONE)

    def mm_tn(self, H, G):
        return ops.gemm_tn(H, G)

    def mm_acc(self, X, W, out, trans_w=False):
        """out += X @ W (or X @ W.T): the accumulating product of the SUMMA stages."""
        return ops.gemm_nn(X, W, trans_w, ops.EPI_ACCUMULATE, out=out)

    def mm_tn_acc(self, H, G, out):
        """out += H.T @ G."""
        return ops.gemm_tn(H, G, out=out, accumulate=True)

    # ---- sparse blocks on the wire: one int32 buffer [rowptr | col | value bits]
    def block_nnz(self, blk):
        return blk.nnz

    def block_to_wire(self, blk):
        return torch.cat([blk.rowptr, blk.col, blk.val.view(torch.int32)])

    def wire_buffer(self, n, nnz):
        return torch.empty(n + 1 + 2 * nnz, dtype=torch.int32, device=self.device)

    def block_from_wire(self, buf, n, m, nnz, reused=False):
        """A received block.  `reused`: the caller keeps it across epochs, so the one-off search for a dense core
        pays; a block that lives for one multiply only gets its hub-row list."""
        blk = ops.CsrBlock(buf[:n + 1], buf[n + 1:n + 1 + nnz], buf[n + 1 + nnz:].view(torch.float32), n, m)
        blk.build_plan(core=bool(reused))
        return blk

    # ---- row-wise pieces of a log-softmax split by columns over a process row
    def row_max(self, z):
        return ops.row_reduce(z, ops.ROW_MAX)

    def row_sum(self, z):
        return ops.row_reduce(z, ops.ROW_SUM)

    def row_sumexp(self, z, ref):
        return ops.row_reduce(z, ops.ROW_SUMEXP, ref)

    def log_softmax_apply(self, z, row_max, row_sum):
        return ops.log_softmax_apply(z, row_max, row_sum)

    def log_softmax_bwd_apply(self, logp, g, row_sum_g):
        return ops.log_softmax_bwd_apply(logp, g, row_sum_g)

    def vector(self, n):
        return torch.empty(n, dtype=torch.float32, device=self.device)

    def zero_matrix_like_weight(self, k, n):
        return torch.zeros((k, n), dtype=torch.float32, device=self.device)

    def act(self, z, act):
        if act == ACT_RELU:
            return ops.relu(z)
        if act == ACT_LOG_SOFTMAX:
            return ops.log_softmax(z)
        return z

    def act_bwd(self, out, g, act):
        """Gradient w.r.t. the pre-activation given the activation OUTPUT `out` and upstream g."""
        if act == ACT_RELU:
            return ops.relu_bwd(out, g)
        if act == ACT_LOG_SOFTMAX:
            return ops.log_softmax_bwd(out, g)
        return g

    def nll(self, logp, y, mask, count, cls_lo=0, cls_hi=None):
        return ops.nll_masked(logp, y, mask, count, cls_lo, cls_hi)

    def synchronize(self):
        torch.cuda.synchronize(self.device)
