"""CPU checker backend with the interface of `cagnet_b200.backend.CudaBackend` -- TEST INFRASTRUCTURE.

Lets the tests drive the package's distributed schedules over Gloo with CPU tensors: every local
computation here is the plain torch restatement of the corresponding reference call (torch.sparse.mm for
`spmm_gpu`, torch.mm for the dense products, F.relu / F.log_softmax and their autograd derivatives).
The product never imports this module.
"""
import torch
import torch.nn.functional as F


class _CpuBlock:
    def __init__(self, rows, cols, vals, n, m):
        self.n, self.m, self.nnz = int(n), int(m), int(vals.numel())
        self.rows, self.cols, self.vals = rows.long(), cols.long(), vals.float()
        self.mat = torch.sparse_coo_tensor(torch.stack([self.rows, self.cols]), self.vals, (self.n, self.m)).coalesce()


class CpuBackend:
    name = "cpu-oracle"
    device = torch.device("cpu")

    def make_block(self, block):
        return _CpuBlock(block.rows, block.cols, block.vals, block.n_rows, block.n_cols)

    def block_nnz(self, blk):
        return blk.nnz

    def block_to_wire(self, blk):
        rowptr = torch.searchsorted(blk.rows.contiguous(), torch.arange(blk.n + 1)).int()
        return torch.cat([rowptr, blk.cols.int(), blk.vals.view(torch.int32)])

    def wire_buffer(self, n, nnz):
        return torch.zeros(n + 1 + 2 * nnz, dtype=torch.int32)

    def block_from_wire(self, buf, n, m, nnz, reused=False):
        rowptr = buf[:n + 1].long()
        rows = torch.repeat_interleave(torch.arange(n), rowptr[1:] - rowptr[:-1])
        return _CpuBlock(rows, buf[n + 1:n + 1 + nnz], buf[n + 1 + nnz:].clone().view(torch.float32), n, m)

    def block_shape(self, blk):
        return blk.n, blk.m

    def spmm(self, blk, B, C, beta):
        prod = torch.sparse.mm(blk.mat, B)            # sparse_coo_tensor.cu:215-226 (alpha = 1)
        if beta:
            C.add_(prod)                              # beta = 1: C += A.B
        else:
            C.copy_(prod)
        return C

    def empty(self, n, f):
        return torch.full((n, f), float("nan"))       # poison: a schedule must never read what it did not write

    def zeros(self, n, f):
        return torch.zeros(n, f)

    def as_matrix(self, x):
        return x.detach().float().contiguous()

    def wire(self, x):
        assert x.is_contiguous()
        return x

    def mm(self, X, W, act="none"):
        return self.act(X @ W, act)

    def mm_nt(self, X, W):
        return X @ W.t()

    def mm_tn(self, H, G):
        return H.t() @ G

    def mm_acc(self, X, W, out, trans_w=False):
        out.add_(X @ (W.t() if trans_w else W))
        return out

    def mm_tn_acc(self, H, G, out):
        out.add_(H.t() @ G)
        return out

    def row_max(self, z):
        return z.max(dim=1)[0] if z.size(1) else torch.full((z.size(0),), float("-inf"))

    def row_sum(self, z):
        return z.sum(dim=1)

    def row_sumexp(self, z, ref):
        return torch.exp(z - ref.unsqueeze(1)).sum(dim=1)

    def log_softmax_apply(self, z, row_max, row_sum):
        return z - row_max.unsqueeze(1) - torch.log(row_sum).unsqueeze(1)

    def log_softmax_bwd_apply(self, logp, g, row_sum_g):
        return g - torch.exp(logp) * row_sum_g.unsqueeze(1)

    def vector(self, n):
        return torch.empty(n)

    def zero_matrix_like_weight(self, k, n):
        return torch.zeros(k, n)

    def act(self, z, act):
        if act == "relu":
            return F.relu(z)
        if act == "log_softmax":
            return F.log_softmax(z, dim=1)
        return z

    def act_bwd(self, out, g, act):
        if act == "relu":
            return g * (out > 0).float()
        if act == "log_softmax":
            return g - torch.exp(out) * g.sum(dim=1, keepdim=True)
        return g

    def nll(self, logp, y, mask, count, cls_lo=0, cls_hi=None):
        n, N = logp.shape
        cls_hi = cls_lo + N if cls_hi is None else cls_hi
        sel = mask.bool() & (y >= cls_lo) & (y < cls_hi)
        rows = torch.nonzero(sel).squeeze(1)
        cols = y[rows] - cls_lo
        loss = -logp[rows, cols].sum() / count
        grad = torch.zeros_like(logp)
        grad[rows, cols] = -1.0 / count
        return loss, grad

    def synchronize(self):
        pass


class PaddedCpuBackend(CpuBackend):
    """The same checker, but every matrix it hands out uses the product's padded row-major layout
    (`cagnet_b200.ops.pad_ld`) with NaN in the pad columns, and `wire()` returns the padded buffer as the CUDA
    backend does.  Run over Gloo it catches what a contiguous CPU tensor hides: a schedule that sends a view of
    the wrong size, slices a padded matrix as if it were dense, or lets pad columns leak into real ones."""
    name = "cpu-oracle-padded"

    @staticmethod
    def _padded_nan(n, f):
        from cagnet_b200 import ops
        ld = ops.pad_ld(f)
        flat = torch.full((max(n * ld, 1),), float("nan"))
        return ops._alias(flat, 0, (n, f), (ld, 1))

    @classmethod
    def _to_padded(cls, x):
        out = cls._padded_nan(x.size(0), x.size(1))
        out.copy_(x)
        return out

    @staticmethod
    def _is_padded(x):
        from cagnet_b200 import ops
        if x.dim() != 2 or x.dtype != torch.float32:
            return False
        if x.size(0) > 1 and x.stride(0) != ops.pad_ld(x.size(1)):
            return False
        if x.size(1) > 1 and x.stride(1) != 1:
            return False
        if x.storage_offset() % ops.pad_ld(x.size(1)) != 0:
            return False
        try:
            ops.base_buffer(x)
        except RuntimeError:
            return False
        return True

    def empty(self, n, f):
        return self._padded_nan(n, f)

    def zeros(self, n, f):
        z = self._padded_nan(n, f)
        z.zero_()
        return z

    def as_matrix(self, x):
        x = x.detach()
        return x if self._is_padded(x) else self._to_padded(x.float())

    def wire(self, x):
        from cagnet_b200 import ops
        return ops.base_buffer(x)

    def spmm(self, blk, B, C, beta):
        prod = torch.sparse.mm(blk.mat, B.contiguous())
        if beta:
            C.add_(prod)
        else:
            C.copy_(prod)
        return C

    def mm(self, X, W, act="none"):
        return self._to_padded(super().mm(X.contiguous(), W, act))

    def mm_nt(self, X, W):
        return self._to_padded(X.contiguous() @ W.t())

    def mm_tn(self, H, G):
        return H.contiguous().t() @ G.contiguous()

    def act(self, z, act):
        return self._to_padded(super().act(z.contiguous(), act))

    def act_bwd(self, out, g, act):
        return self._to_padded(super().act_bwd(out.contiguous(), g.contiguous(), act))

    def log_softmax_apply(self, z, row_max, row_sum):
        return self._to_padded(super().log_softmax_apply(z.contiguous(), row_max, row_sum))

    def log_softmax_bwd_apply(self, logp, g, row_sum_g):
        return self._to_padded(super().log_softmax_bwd_apply(logp.contiguous(), g.contiguous(), row_sum_g))

    def nll(self, logp, y, mask, count, cls_lo=0, cls_hi=None):
        loss, grad = super().nll(logp.contiguous(), y, mask, count, cls_lo, cls_hi)
        return loss, self._to_padded(grad)
