"""2D (SUMMA) full-batch GCN training on a q x q process grid, q = floor(sqrt(P)).

Host-side mirror of the reference's `gcn_distr_2d.py`: same grid (`rank = row*q + col`), same block
ownership (A and H by rows AND columns), same stage order and sources for the sparse SUMMA
(`summa_sparse`), the local-weight SUMMA (`summa_loc`), the pairwise transpose and the dense SUMMA
(`summa`), the row-distributed log-softmax and the class-column-restricted loss.

What changes underneath:
  * A blocks travel as int32 CSR (offsets | columns | value bits) in one broadcast and are cached by the
    receivers after the first epoch (the adjacency is static); the reference re-sends every block every
    epoch as a 3 x nnz fp32 tensor and round-trips the indices through fp32 (gcn_distr_2d.py:362-383).
    `cache_blocks=False` restores the per-epoch broadcast.
  * the block sizes of every rank are exchanged once at set-up, so no stage needs a host synchronisation
    (`.item()` at gcn_distr_2d.py:357).
  * log-softmax backward needs one all-reduce of a per-row scalar instead of gathering full-width rows
    (gcn_distr_2d.py:570-645).
  * H^T is never materialised: the transposed block is exchanged untransposed and the product kernel reads
    it as H^T.
"""
import torch
import torch.distributed as dist
import torch.nn.functional as F

from . import partition
from .backend import ACT_LOG_SOFTMAX, ACT_NONE, ACT_RELU
from .dist1d import Data, act_name  # noqa: F401  (Data re-exported for callers of this module)
from .timing import CATEGORIES_2D, Timers, all_gather_bytes, all_reduce_bytes


class Runtime:
    def __init__(self, backend, activations=True, normalization=True, timing=False, overlap=True, cache_blocks=True,
                 reference_label_alignment=True, directed=False):
        self.backend = backend
        self.activations = bool(activations)
        self.normalization = bool(normalization)
        self.overlap = bool(overlap)
        self.cache_blocks = bool(cache_blocks)
        self.reference_label_alignment = bool(reference_label_alignment)
        # backward pass multiplies by blocks of A^T instead of reusing A's (which is exact for undirected graphs
        # only, gcn_distr_2d.py:683): a second set of adjacency blocks per process
        self.directed = bool(directed)
        self.timers = Timers(CATEGORIES_2D, timing, getattr(backend, "synchronize", None))


class Grid:
    """Process grid and communicators (gcn_distr_2d.py:516-535, 1179-1207)."""

    def __init__(self, rank, size):
        self.rank, self.size = rank, size
        self.q = partition.grid_side_2d(size)
        self.row, self.col = rank // self.q, rank % self.q
        self.active = rank < self.q * self.q
        self.rank_t = self.col * self.q + self.row
        self.comm = dist.is_initialized() and size > 1
        self.group = self.row_groups = self.col_groups = None
        if self.comm:
            self.group = dist.new_group(list(range(self.q * self.q)))      # the processes that hold a block
            rows, cols = partition.proc_groups_2d(size)
            self.row_groups = [dist.new_group(r) for r in rows]
            self.col_groups = [dist.new_group(c) for c in cols]

    @property
    def row_group(self):
        return self.row_groups[self.row] if self.comm else None

    @property
    def col_group(self):
        return self.col_groups[self.col] if self.comm else None


class AdjOperator:
    """One process's block of a sparse operator and what the stage loop keeps with it: the wire form it
    broadcasts, the blocks received from the other processes of its row (kept after the first product), and the
    nonzero count of every process's block (exchanged once, so that receive buffers can be sized)."""

    def __init__(self, be, block, rank, count, group, device):
        self.adj_block = be.make_block(block)
        self.adj_wire = be.block_to_wire(self.adj_block) if group is not None else None
        self.block_cache, self.blocks_sent = {}, False
        nnz = torch.zeros(count, dtype=torch.int64)
        nnz[rank] = be.block_nnz(self.adj_block)
        if group is not None:
            nnz = nnz.to(device)
            dist.all_reduce(nnz, group=group)
        self.nnz_of = [int(v) for v in nnz.tolist()]


def _offsets(sizes):
    out = [0]
    for s in sizes:
        out.append(out[-1] + s)
    return out


def _bcast(tensor, src, group, async_op=False):
    return dist.broadcast(tensor, src=src, group=group, async_op=async_op)


# ------------------------------------------------------------------------------------------ SUMMA pieces
def summa_sparse(model, inputs, op=None):
    """Z[row, col] = sum_k A[row, k] . H[k, col]   (gcn_distr_2d.py:286-426).

    Stage k: process (row, k) supplies A[row, k] to its process row, process (k, col) supplies H[k, col] to its
    process column.  The H broadcast of stage k+1 is posted before the multiply of stage k is queued."""
    rt, g, be = model.rt, model.grid, model.rt.backend
    op = model if op is None else op          # whose block, wire form, cache and counts the stages use
    q = g.q
    inputs = be.as_matrix(inputs)
    f_col = inputs.size(1)
    z = be.empty(model.row_sizes[g.row], f_col)
    bufs = [None, None]

    def a_block(k):
        src = g.row * q + k
        if src == g.rank:
            blk = op.adj_block
            if g.comm and not (rt.cache_blocks and op.blocks_sent):
                with rt.timers.comm("a_block_broadcast", op.adj_wire.numel() * 4, "comm_time", "summa_sparse_bcast1"):
                    _bcast(op.adj_wire, src, g.row_group)
                rt.timers.count("summa_sparse_bcast1_words", op.adj_wire.numel())
            return blk
        if rt.cache_blocks and k in op.block_cache:
            return op.block_cache[k]
        n_r, n_c, nnz = model.row_sizes[g.row], model.row_sizes[k], op.nnz_of[src]
        buf = be.wire_buffer(n_r, nnz)
        with rt.timers.comm("a_block_broadcast", buf.numel() * 4, "comm_time", "summa_sparse_bcast1"):
            _bcast(buf, src, g.row_group)
        rt.timers.count("summa_sparse_bcast1_words", buf.numel())
        blk = be.block_from_wire(buf, n_r, n_c, nnz, reused=rt.cache_blocks)
        if rt.cache_blocks:
            op.block_cache[k] = blk
        return blk

    def post_h(k):
        src = k * q + g.col
        rows = model.row_sizes[k]
        if src == g.rank:
            tensor = inputs
        else:
            if bufs[k % 2] is None:
                bufs[k % 2] = be.empty(max(model.row_sizes), f_col)
            tensor = bufs[k % 2][:rows]
        rt.timers.count("summa_sparse_bcast2_words", rows * f_col)
        if g.comm:
            rt.timers.traffic("h_broadcast", be.wire(tensor).numel() * 4)
        work = _bcast(be.wire(tensor), src, g.col_group, async_op=True) if g.comm else None
        return tensor, work

    serial = rt.timers.enabled or not rt.overlap
    pending = None
    for k in range(q):
        blk = a_block(k)
        if serial:
            with rt.timers.region("comm_time", "summa_sparse_bcast2", "link:h_broadcast"):
                tensor, work = post_h(k)
                if work is not None:
                    work.wait()
        else:
            tensor, work = pending if pending is not None else post_h(k)
            pending = post_h(k + 1) if k + 1 < q else None
            if work is not None:
                work.wait()
        with rt.timers.region("comp_time", "summa_sparse_comp"):
            be.spmm(blk, tensor, z, 0.0 if k == 0 else 1.0)
    op.blocks_sent = True
    return z


def summa_loc(model, mata, weight, transposed):
    """Z[row, col] = sum_k M[row, k] . W[k, col] with W replicated (gcn_distr_2d.py:428-514): only the left
    operand's blocks travel, along the process row; every process slices its own W[k, col].
    transposed=True multiplies by weight.t() (the grad_input product, gcn_distr_2d.py:841)."""
    rt, g, be = model.rt, model.grid, model.rt.backend
    q = g.q
    mata = be.as_matrix(mata)
    w = weight.detach()
    k_sizes = partition.chunk_sizes(w.size(1) if transposed else w.size(0), q)     # split of the contracted dim
    o_sizes = partition.chunk_sizes(w.size(0) if transposed else w.size(1), q)     # split of the output dim
    ko, oo = _offsets(k_sizes), _offsets(o_sizes)
    n_r = model.row_sizes[g.row]
    z = None
    for k in range(q):
        src = g.row * q + k
        if src == g.rank:
            acol = mata
        else:
            acol = be.empty(n_r, k_sizes[k])
        if g.comm:
            with rt.timers.comm("z_block_broadcast", be.wire(acol).numel() * 4, "comm_time", "summa_loc_bcast"):
                _bcast(be.wire(acol), src, g.row_group)
        if transposed:
            part = w[oo[g.col]:oo[g.col + 1], ko[k]:ko[k + 1]]       # used transposed: (out chunk) x (k chunk)
        else:
            part = w[ko[k]:ko[k + 1], oo[g.col]:oo[g.col + 1]]
        with rt.timers.region("comp_time"):
            if z is None:
                z = be.mm_nt(acol, part) if transposed else be.mm(acol, part)
            else:
                be.mm_acc(acol, part, z, trans_w=transposed)
    return z


def transpose(model, mat, total_width):
    """Pairwise exchange with the mirror process (col, row): returns the mirror's block, UNtransposed
    (gcn_distr_2d.py:133-182 sends mat.t(); the product kernel below reads the block as its transpose)."""
    g, be = model.grid, model.rt.backend
    mat = be.as_matrix(mat)
    if g.rank == g.rank_t or not g.comm:
        return mat
    f_sizes = partition.chunk_sizes(total_width, g.q)
    recv = be.empty(model.row_sizes[g.col], f_sizes[g.row])
    ops = [dist.P2POp(dist.isend, be.wire(mat), g.rank_t), dist.P2POp(dist.irecv, be.wire(recv), g.rank_t)]
    with model.rt.timers.comm("transpose_exchange", be.wire(recv).numel() * 4):
        for work in dist.batch_isend_irecv(ops):
            work.wait()
    return recv


def summa_tn(model, ht, ag, f_in, f_out):
    """grad_W[row, col] = sum_k H[k, row]^T . AG[k, col]   (the dense SUMMA, gcn_distr_2d.py:184-284, with
    `ht` = this process's transposed-position block H[col, row], still row-major n_col x f_row)."""
    rt, g, be = model.rt, model.grid, model.rt.backend
    q = g.q
    f_sizes, o_sizes = partition.chunk_sizes(f_in, q), partition.chunk_sizes(f_out, q)
    ag = be.as_matrix(ag)
    z = be.zero_matrix_like_weight(f_sizes[g.row], o_sizes[g.col])
    for k in range(q):
        row_src, col_src = g.row * q + k, k * q + g.col
        n_k = model.row_sizes[k]
        acol = ht if row_src == g.rank else be.empty(n_k, f_sizes[g.row])
        brow = ag if col_src == g.rank else be.empty(n_k, o_sizes[g.col])
        if g.comm:
            with rt.timers.comm("grad_w_summa_broadcast", be.wire(acol).numel() * 4, "comm_time", "summa_bcast1"):
                _bcast(be.wire(acol), row_src, g.row_group)
            with rt.timers.comm("grad_w_summa_broadcast", be.wire(brow).numel() * 4, "comm_time", "summa_bcast2"):
                _bcast(be.wire(brow), col_src, g.col_group)
        with rt.timers.region("comp_time", "summa_comp"):
            be.mm_tn_acc(acol, brow, z)
    return z


def gather_weight_blocks(model, block, f_in, f_out):
    """Every process ends up with the whole grad_W: all-gather of the q x q blocks, padded to the largest block
    (gcn_distr_2d.py:862-909, without the sentinel-value trimming: the block sizes are known)."""
    g = model.grid
    q = g.q
    f_sizes, o_sizes = partition.chunk_sizes(f_in, q), partition.chunk_sizes(f_out, q)
    if not g.comm:
        return block
    padded = torch.zeros((max(f_sizes), max(o_sizes)), dtype=block.dtype, device=block.device)
    padded[:block.size(0), :block.size(1)] = block
    parts = [torch.empty_like(padded) for _ in range(q * q)]
    with model.rt.timers.comm("grad_w_all_gather", all_gather_bytes(padded.numel() * 4, q * q)):
        dist.all_gather(parts, padded, group=g.group)
    rows = []
    for i in range(q):
        rows.append(torch.cat([parts[i * q + j][:f_sizes[i], :o_sizes[j]] for j in range(q)], dim=1))
    return torch.cat(rows, dim=0)


def dist_log_softmax(model, z):
    """Log-softmax of rows whose columns are spread over the process row (gcn_distr_2d.py:537-568)."""
    g, be = model.grid, model.rt.backend
    m = be.row_max(z)
    if g.comm:
        with model.rt.timers.comm("log_softmax_all_reduce", all_reduce_bytes(m.numel() * 4, g.q)):
            dist.all_reduce(m, op=dist.ReduceOp.MAX, group=g.row_group)
    s = be.row_sumexp(z, m)
    if g.comm:
        with model.rt.timers.comm("log_softmax_all_reduce", all_reduce_bytes(s.numel() * 4, g.q)):
            dist.all_reduce(s, op=dist.ReduceOp.SUM, group=g.row_group)
    return be.log_softmax_apply(z, m, s)


def dist_log_softmax_bwd(model, logp, grad):
    """dZ = G - softmax . rowsum(G), the row sum taken over the whole process row."""
    g, be = model.grid, model.rt.backend
    rs = be.row_sum(grad)
    if g.comm:
        with model.rt.timers.comm("log_softmax_all_reduce", all_reduce_bytes(rs.numel() * 4, g.q)):
            dist.all_reduce(rs, op=dist.ReduceOp.SUM, group=g.row_group)
    return be.log_softmax_bwd_apply(logp, grad, rs)


# ------------------------------------------------------------------------------------------ layer
class GCNFunc(torch.autograd.Function):
    """gcn_distr_2d.py:647-918."""

    @staticmethod
    def forward(ctx, inputs, weight, model, func):
        rt, be = model.rt, model.rt.backend
        act = act_name(func) if rt.activations else ACT_NONE
        z = summa_sparse(model, inputs)
        z = summa_loc(model, z, weight, transposed=False)
        if act == ACT_LOG_SOFTMAX:
            out = dist_log_softmax(model, z)
        elif act == ACT_RELU:
            out = be.act(z, ACT_RELU)
        else:
            out = z
        ctx.save_for_backward(inputs, weight, out)
        ctx.model, ctx.act = model, act
        return out

    @staticmethod
    def backward(ctx, grad_output):
        inputs, weight, out = ctx.saved_tensors
        model, act = ctx.model, ctx.act
        rt, be = model.rt, model.rt.backend
        grad_output = be.as_matrix(grad_output)
        if act == ACT_LOG_SOFTMAX:
            dz = dist_log_softmax_bwd(model, out, grad_output)
        elif act == ACT_RELU:
            dz = be.act_bwd(out, grad_output, ACT_RELU)
        else:
            dz = grad_output
        # A is used as its own transpose: exact for undirected graphs only (gcn_distr_2d.py:683); a model built
        # with `directed` holds the blocks of A^T and multiplies by those
        ag = summa_sparse(model, dz, model.adj_t)
        grad_input = summa_loc(model, ag, weight, transposed=True) if ctx.needs_input_grad[0] else None
        with rt.timers.region("transpose_time"):
            ht = transpose(model, inputs, weight.size(0))
        block = summa_tn(model, ht, ag, weight.size(0), weight.size(1))
        grad_weight = gather_weight_blocks(model, block, weight.size(0), weight.size(1))
        return grad_input, grad_weight, None, None


class MaskedNLL(torch.autograd.Function):
    @staticmethod
    def forward(ctx, outputs, model):
        be = model.rt.backend
        loss, grad = be.nll(be.as_matrix(outputs), model.y_eff, model.mask_eff, model.train_count_global,
                            model.cls_lo, model.cls_hi)
        ctx.grad, ctx.wire = grad, be.wire
        return loss

    @staticmethod
    def backward(ctx, g):
        ctx.wire(ctx.grad).mul_(g)
        return ctx.grad, None


class Model:
    """One process's share: its A block (cached CSR), H block, labels/mask slice and class range."""

    def __init__(self, rt, rank, size, inputs, adj_matrix, data, features, classes, grid=None):
        be = rt.backend
        self.rt, self.rank, self.size, self.features, self.classes = rt, rank, size, features, classes
        self.grid = g = grid if grid is not None else Grid(rank, size)
        q = g.q
        n = inputs.size(0)
        self.node_count = n
        self.row_sizes = partition.chunk_sizes(n, q)
        everyone = g.group if (g.comm and q * q == size) else None
        inputs_loc, block = partition.twod_partition(rank, size, inputs, adj_matrix, rt.normalization,
                                                     degree_group=everyone)
        self.inputs_loc = be.as_matrix(inputs_loc)
        self.adj_block = be.make_block(block)
        self.adj_wire = be.block_to_wire(self.adj_block) if g.comm else None
        self.block_cache, self.blocks_sent = {}, False
        nnz = torch.zeros(q * q, dtype=torch.int64)
        nnz[rank] = be.block_nnz(self.adj_block)
        if g.comm:
            nnz = nnz.to(self.inputs_loc.device)
            dist.all_reduce(nnz, group=g.group)
        self.nnz_of = [int(v) for v in nnz.tolist()]
        self.adj_t = None
        if rt.directed:
            _, block_t = partition.twod_partition(rank, size, inputs, adj_matrix, rt.normalization,
                                                  degree_group=everyone, transposed=True)
            self.adj_t = AdjOperator(be, block_t, rank, q * q, g.group if g.comm else None, self.inputs_loc.device)
        self._setup_labels(data, n, classes)

    def _setup_labels(self, data, n, classes):
        """Labels and mask as the reference's loss sees them (gcn_distr_2d.py:942-970): the slice
        split(., L)[rank_row] with L this process's row count, compressed to the train rows, position p of
        the compressed list paired with local output row p; the class range of this process column without
        the remainder on the last column (gcn_distr_2d.py:947-952)."""
        g, rt = self.grid, self.rt
        dev = self.inputs_loc.device
        L = self.row_sizes[g.row]
        mask_all = data.train_mask.bool()
        if rt.reference_label_alignment:
            lo = min(n, g.row * L)
            hi = min(n, lo + L)
            y_s, m_s = data.y[lo:hi].long(), mask_all[lo:hi]
            comp = y_s[m_s]
            y_eff = torch.zeros(L, dtype=torch.int64, device=comp.device)
            m_eff = torch.zeros(L, dtype=torch.bool, device=comp.device)
            y_eff[:comp.numel()] = comp
            m_eff[:comp.numel()] = True
        else:
            r0 = sum(self.row_sizes[:g.row])
            y_eff, m_eff = data.y[r0:r0 + L].long(), mask_all[r0:r0 + L]
        self.y_eff, self.mask_eff = y_eff.to(dev), m_eff.to(dev)
        self.train_count_global = int(mask_all.sum())
        self.local_train_rows = int(m_eff.sum())
        per = classes // g.q
        self.cls_lo = g.col * per
        if rt.reference_label_alignment:
            self.cls_hi = min((g.col + 1) * per, classes)
        else:
            self.cls_hi = classes if g.col == g.q - 1 else (g.col + 1) * per

    def init_weights(self, mid_layer):
        torch.manual_seed(0)
        dev = self.inputs_loc.device
        self.weight1 = torch.nn.Parameter(torch.rand(self.features, mid_layer).to(dev))
        self.weight2 = torch.nn.Parameter(torch.rand(mid_layer, self.classes).to(dev))
        self.optimizer = torch.optim.Adam([self.weight1, self.weight2], lr=0.01)
        return self.weight1, self.weight2

    def train(self):
        return train(self)


def train(model):
    """gcn_distr_2d.py:920-1001."""
    rt = model.rt
    outputs = GCNFunc.apply(model.inputs_loc, model.weight1, model, F.relu)
    outputs = GCNFunc.apply(outputs, model.weight2, model, F.log_softmax)
    model.optimizer.zero_grad()
    if model.local_train_rows > 0:
        with rt.timers.region("loss_calc_time"):
            loss = MaskedNLL.apply(outputs, model)
        loss.backward()
        model.last_loss = loss.detach()
    else:
        outputs.backward(rt.backend.zeros(outputs.size(0), outputs.size(1)))
        model.last_loss = torch.zeros((), device=outputs.device)
    model.optimizer.step()
    return outputs
