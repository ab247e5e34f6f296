"""3D (split-3D-SpMM) full-batch GCN training on a q x q x c process grid with q = c = cbrt(P).

Host-side mirror of the reference's `gcn_distr_3d.py`: rank = i*(q*c) + j*c + k; process (i, j, k) owns
column slab k of adjacency block (i, j) and row chunk k of feature block (i, j); a sparse product is a 2D
SUMMA inside each layer k over its slab followed by an all-reduce along the fiber (i, j, .) and a re-split
(`split3dspmm_sparse`, gcn_distr_3d.py:325-500); the product with the replicated weight
(`split3dspmm_loc`, :503-627) and the weight-gradient product (`split3dspmm_dense`, :178-323) follow the same
pattern.  The reference model is linear and unnormalised (its activations are commented out,
gcn_distr_3d.py:837-843, and `normalization` is a constant False, :66); `activations` / `normalization` are
this package's extensions and default to the reference behaviour.

Differences underneath (same results): CSR slabs cached after the first epoch, slab sizes exchanged once at
set-up, one fiber all-reduce per weight product instead of one per stage (the sum is linear), and the
transposed operand of the weight-gradient product is exchanged untransposed.
"""
import torch
import torch.distributed as dist
import torch.nn.functional as F

from . import partition
from .backend import ACT_LOG_SOFTMAX, ACT_NONE, ACT_RELU
from .dist1d import Data, act_name  # noqa: F401
from .dist2d import AdjOperator, MaskedNLL, _bcast, _offsets
from .timing import CATEGORIES_3D, Timers, all_gather_bytes, all_reduce_bytes


class Runtime:
    def __init__(self, backend, activations=False, normalization=False, timing=False, overlap=True, cache_blocks=True,
                 reference_label_alignment=True, directed=False):
        self.backend = backend
        self.activations = bool(activations)
        self.normalization = bool(normalization)
        self.overlap = bool(overlap)
        self.cache_blocks = bool(cache_blocks)
        self.reference_label_alignment = bool(reference_label_alignment)
        self.directed = bool(directed)         # backward pass over slabs of A^T (the reference reuses A's)
        self.timers = Timers(CATEGORIES_3D, timing, getattr(backend, "synchronize", None))


class Grid:
    """gcn_distr_3d.py:629-672, 754-756."""

    def __init__(self, rank, size):
        self.rank, self.size = rank, size
        self.q = q = partition.grid_side_3d(size)
        self.i, self.j, self.k = partition.coords_3d(rank, q)
        self.comm = dist.is_initialized() and size > 1
        self.group = None
        self._rows = self._cols = self._fibers = None
        if self.comm:
            self.group = dist.new_group(list(range(size)))
            rows, cols, fibers = partition.proc_groups_3d(size)
            self._rows = [[dist.new_group(r) for r in per_k] for per_k in rows]
            self._cols = [[dist.new_group(c) for c in per_k] for per_k in cols]
            self._fibers = [dist.new_group(f) for f in fibers]

    def rank_of(self, i, j, k):
        return i * self.q * self.q + j * self.q + k

    @property
    def row_group(self):          # same i and k, j varies
        return self._rows[self.i][self.k] if self.comm else None

    @property
    def col_group(self):          # same j and k, i varies
        return self._cols[self.j][self.k] if self.comm else None

    @property
    def fiber_group(self):        # same i and j, k varies
        return self._fibers[self.rank // self.q] if self.comm else None


def _column_chunk(be, z, sizes, k):
    off = _offsets(sizes)
    return be.as_matrix(z[:, off[k]:off[k + 1]])


def split3dspmm_sparse(model, inputs, op=None):
    """(A . H) block (i, j), column chunk k.  gcn_distr_3d.py:325-500."""
    rt, g, be = model.rt, model.grid, model.rt.backend
    op = model if op is None else op          # whose block, wire form, cache and counts the stages use
    q = g.q
    inputs = be.as_matrix(inputs)
    f_j = inputs.size(1)
    z = be.empty(model.row_sizes[g.i], f_j)
    bufs = [None, None]

    def a_slab(kp):
        src = g.rank_of(g.i, kp, g.k)
        if src == g.rank:
            if g.comm and not (rt.cache_blocks and op.blocks_sent):
                with rt.timers.comm("a_block_broadcast", op.adj_wire.numel() * 4, "comm_time", "summa_sparse_bcast1"):
                    _bcast(op.adj_wire, src, g.row_group)
                rt.timers.count("summa_sparse_bcast1_words", op.adj_wire.numel())
            return op.adj_block
        if rt.cache_blocks and kp in op.block_cache:
            return op.block_cache[kp]
        n_r, n_c, nnz = model.row_sizes[g.i], model.sub_sizes[kp][g.k], op.nnz_of[src]
        buf = be.wire_buffer(n_r, nnz)
        with rt.timers.comm("a_block_broadcast", buf.numel() * 4, "comm_time", "summa_sparse_bcast1"):
            _bcast(buf, src, g.row_group)
        rt.timers.count("summa_sparse_bcast1_words", buf.numel())
        blk = be.block_from_wire(buf, n_r, n_c, nnz, reused=rt.cache_blocks)
        if rt.cache_blocks:
            op.block_cache[kp] = blk
        return blk

    def post_h(kp):
        src = g.rank_of(kp, g.j, g.k)
        rows = model.sub_sizes[kp][g.k]
        if src == g.rank:
            tensor = inputs
        else:
            if bufs[kp % 2] is None:
                bufs[kp % 2] = be.empty(model.max_sub, f_j)
            tensor = bufs[kp % 2][:rows]
        rt.timers.count("summa_sparse_bcast2_words", rows * f_j)
        if g.comm:
            rt.timers.traffic("h_broadcast", be.wire(tensor).numel() * 4)
        work = _bcast(be.wire(tensor), src, g.col_group, async_op=True) if g.comm else None
        return tensor, work

    serial = rt.timers.enabled or not rt.overlap
    pending = None
    for kp in range(q):
        blk = a_slab(kp)
        if serial:
            with rt.timers.region("comm_time", "summa_sparse_bcast2", "link:h_broadcast"):
                tensor, work = post_h(kp)
                if work is not None:
                    work.wait()
        else:
            tensor, work = pending if pending is not None else post_h(kp)
            pending = post_h(kp + 1) if kp + 1 < q else None
            if work is not None:
                work.wait()
        with rt.timers.region("comp_time", "summa_sparse_comp"):
            be.spmm(blk, tensor, z, 0.0 if kp == 0 else 1.0)
    op.blocks_sent = True
    if g.comm:
        with rt.timers.comm("z_fiber_all_reduce", all_reduce_bytes(be.wire(z).numel() * 4, q), "comm_time",
                            "summa_sparse_reduce"):
            dist.all_reduce(be.wire(z), group=g.fiber_group)
    return _column_chunk(be, z, partition.chunk_sizes(f_j, q), g.k)


def split3dspmm_loc(model, mata, weight, transposed):
    """(M . W) block (i, j), row chunk k, for M held as column chunks and W replicated.
    gcn_distr_3d.py:503-627; the contracted dimension is split q ways and each part c ways, the fiber sum is
    taken once after the stage loop."""
    rt, g, be = model.rt, model.grid, model.rt.backend
    q = g.q
    mata = be.as_matrix(mata)
    w = weight.detach()
    k_total = w.size(1) if transposed else w.size(0)
    o_total = w.size(0) if transposed else w.size(1)
    k_sizes = [partition.chunk_sizes(s, q) for s in partition.chunk_sizes(k_total, q)]    # [k'][k]
    flat = [s for per in k_sizes for s in per]
    ko = _offsets(flat)
    oo = _offsets(partition.chunk_sizes(o_total, q))
    n_i = model.row_sizes[g.i]
    z = None
    for kp in range(q):
        src = g.rank_of(g.i, kp, g.k)
        acol = mata if src == g.rank else be.empty(n_i, k_sizes[kp][g.k])
        if g.comm:
            with rt.timers.comm("z_block_broadcast", be.wire(acol).numel() * 4, "comm_time", "summa_loc_bcast"):
                _bcast(be.wire(acol), src, g.row_group)
        c0, c1 = ko[kp * q + g.k], ko[kp * q + g.k + 1]
        part = w[oo[g.j]:oo[g.j + 1], c0:c1] if transposed else w[c0:c1, oo[g.j]:oo[g.j + 1]]
        with rt.timers.region("comp_time", "summa_comp"):
            if z is None:
                z = be.mm_nt(acol, part) if transposed else be.mm(acol, part)
            else:
                be.mm_acc(acol, part, z, trans_w=transposed)
    if g.comm:
        with rt.timers.comm("zw_fiber_all_reduce", all_reduce_bytes(be.wire(z).numel() * 4, q), "comm_time",
                            "summa_reduce"):
            dist.all_reduce(be.wire(z), group=g.fiber_group)
    ro = _offsets(model.sub_sizes[g.i])
    return be.as_matrix(z[ro[g.k]:ro[g.k + 1]])


def transpose(model, ag, out_total):
    """Row chunk k of the mirror block AG[j, i], left untransposed: all-gather the column chunks along the fiber,
    then exchange row chunk k with process (j, i, k).  gcn_distr_3d.py:105-176."""
    g, be = model.grid, model.rt.backend
    q = g.q
    ag = be.as_matrix(ag)
    o_sizes = partition.chunk_sizes(out_total, q)
    n_i = model.row_sizes[g.i]
    if g.comm:
        widths = partition.chunk_sizes(o_sizes[g.j], q)
        padded = torch.zeros((n_i, max(widths)), dtype=torch.float32, device=ag.device)
        padded[:, :ag.size(1)] = ag
        parts = [torch.empty_like(padded) for _ in range(q)]
        with model.rt.timers.comm("transpose_all_gather", all_gather_bytes(padded.numel() * 4, q)):
            dist.all_gather(parts, padded, group=g.fiber_group)
        full = torch.cat([parts[k][:, :widths[k]] for k in range(q)], dim=1)
    else:
        full = ag
    ro = _offsets(model.sub_sizes[g.i])
    mine = be.as_matrix(full[ro[g.k]:ro[g.k + 1]])
    if g.i == g.j or not g.comm:
        return mine
    peer = g.rank_of(g.j, g.i, g.k)
    recv = be.empty(model.sub_sizes[g.j][g.k], o_sizes[g.i])
    ops = [dist.P2POp(dist.isend, be.wire(mine), peer), dist.P2POp(dist.irecv, be.wire(recv), peer)]
    with model.rt.timers.comm("transpose_exchange", be.wire(recv).numel() * 4):
        for work in dist.batch_isend_irecv(ops):
            work.wait()
    return recv


def split3dspmm_tn(model, ag_t, inputs, f_in, f_out):
    """Block (f_in chunk j, f_out chunk i) of H^T . AG: gcn_distr_3d.py:178-323 computes its transpose."""
    rt, g, be = model.rt, model.grid, model.rt.backend
    q = g.q
    inputs = be.as_matrix(inputs)
    f_sizes, o_sizes = partition.chunk_sizes(f_in, q), partition.chunk_sizes(f_out, q)
    z = be.zero_matrix_like_weight(f_sizes[g.j], o_sizes[g.i])
    for kp in range(q):
        row_src, col_src = g.rank_of(g.i, kp, g.k), g.rank_of(kp, g.j, g.k)
        rows = model.sub_sizes[kp][g.k]
        acol = ag_t if row_src == g.rank else be.empty(rows, o_sizes[g.i])
        brow = inputs if col_src == g.rank else be.empty(rows, f_sizes[g.j])
        if g.comm:
            with rt.timers.comm("grad_w_summa_broadcast", be.wire(acol).numel() * 4, "comm_time", "summa_bcast1"):
                _bcast(be.wire(acol), row_src, g.row_group)
            with rt.timers.comm("grad_w_summa_broadcast", be.wire(brow).numel() * 4, "comm_time", "summa_bcast2"):
                _bcast(be.wire(brow), col_src, g.col_group)
        with rt.timers.region("comp_time", "summa_comp"):
            be.mm_tn_acc(brow, acol, z)
    if g.comm:
        with rt.timers.comm("grad_w_fiber_all_reduce", all_reduce_bytes(z.numel() * 4, q), "comm_time", "summa_reduce"):
            dist.all_reduce(z, group=g.fiber_group)
    return z


def gather_weight_blocks(model, block, f_in, f_out):
    """Whole grad_W on every process from the blocks held by the k = 0 layer (gcn_distr_3d.py:984-1049)."""
    g = model.grid
    q = g.q
    if not g.comm:
        return block
    f_sizes, o_sizes = partition.chunk_sizes(f_in, q), partition.chunk_sizes(f_out, q)
    padded = torch.zeros((max(f_sizes), max(o_sizes)), dtype=block.dtype, device=block.device)
    padded[:block.size(0), :block.size(1)] = block
    parts = [torch.empty_like(padded) for _ in range(g.size)]
    with model.rt.timers.comm("grad_w_all_gather", all_gather_bytes(padded.numel() * 4, g.size)):
        dist.all_gather(parts, padded, group=g.group)
    rows = []
    for j in range(q):
        rows.append(torch.cat([parts[g.rank_of(i, j, 0)][:f_sizes[j], :o_sizes[i]] for i in range(q)], dim=1))
    return torch.cat(rows, dim=0)


def dist_log_softmax(model, z):
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
    g, be = model.grid, model.rt.backend
    rs = be.row_sum(grad)
    if g.comm:
        with model.rt.timers.comm("log_softmax_all_reduce", all_reduce_bytes(rs.numel() * 4, g.q)):
            dist.all_reduce(rs, op=dist.ReduceOp.SUM, group=g.row_group)
    return be.log_softmax_bwd_apply(logp, grad, rs)


class GCNFunc(torch.autograd.Function):
    """gcn_distr_3d.py:741-1052."""

    @staticmethod
    def forward(ctx, inputs, weight, model, func):
        rt, be = model.rt, model.rt.backend
        act = act_name(func) if rt.activations else ACT_NONE
        z = split3dspmm_sparse(model, inputs)
        z = split3dspmm_loc(model, z, weight, transposed=False)
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
        ag = split3dspmm_sparse(model, dz, model.adj_t)         # A's own slabs unless the model is `directed`
        grad_input = split3dspmm_loc(model, ag, weight, transposed=True) if ctx.needs_input_grad[0] else None
        with rt.timers.region("transpose_time"):
            ag_t = transpose(model, ag, weight.size(1))
        block = split3dspmm_tn(model, ag_t, inputs, weight.size(0), weight.size(1))
        grad_weight = gather_weight_blocks(model, block, weight.size(0), weight.size(1))
        return grad_input, grad_weight, None, None


class Model:
    def __init__(self, rt, rank, size, inputs, adj_matrix, data, features, classes, grid=None):
        be = rt.backend
        self.rt, self.rank, self.size, self.features, self.classes = rt, rank, size, features, classes
        self.grid = g = grid if grid is not None else Grid(rank, size)
        q = g.q
        n = inputs.size(0)
        self.node_count = n
        self.row_sizes = partition.chunk_sizes(n, q)
        self.sub_sizes = [partition.chunk_sizes(s, q) for s in self.row_sizes]
        self.max_sub = max(max(s) for s in self.sub_sizes)
        inputs_loc, slab = partition.threed_partition(rank, size, inputs, adj_matrix, rt.normalization,
                                                      degree_group=g.group if g.comm else None)
        self.inputs_loc = be.as_matrix(inputs_loc)
        self.adj_block = be.make_block(slab)
        self.adj_wire = be.block_to_wire(self.adj_block) if g.comm else None
        self.block_cache, self.blocks_sent = {}, False
        nnz = torch.zeros(size, dtype=torch.int64)
        nnz[rank] = be.block_nnz(self.adj_block)
        if g.comm:
            nnz = nnz.to(self.inputs_loc.device)
            dist.all_reduce(nnz, group=g.group)
        self.nnz_of = [int(v) for v in nnz.tolist()]
        self.adj_t = None
        if rt.directed:
            _, slab_t = partition.threed_partition(rank, size, inputs, adj_matrix, rt.normalization,
                                                   degree_group=g.group if g.comm else None, transposed=True)
            self.adj_t = AdjOperator(be, slab_t, rank, size, g.group if g.comm else None, self.inputs_loc.device)
        self._setup_labels(data, n, classes)

    def _setup_labels(self, data, n, classes):
        """gcn_distr_3d.py:1080-1108: slice split(., L)[i*c + k] with L this process's row count, compressed to
        the train rows and paired with local rows by position; class range of process column j, the last
        column taking the remainder."""
        g, rt = self.grid, self.rt
        dev = self.inputs_loc.device
        L = self.sub_sizes[g.i][g.k]
        mask_all = data.train_mask.bool()
        if rt.reference_label_alignment:
            lo = min(n, (g.i * g.q + g.k) * L)
            hi = min(n, lo + L)
            y_s, m_s = data.y[lo:hi].long(), mask_all[lo:hi]
            comp = y_s[m_s]
            y_eff = torch.zeros(L, dtype=torch.int64, device=comp.device)
            m_eff = torch.zeros(L, dtype=torch.bool, device=comp.device)
            y_eff[:comp.numel()] = comp
            m_eff[:comp.numel()] = True
        else:
            r0 = sum(self.row_sizes[:g.i]) + sum(self.sub_sizes[g.i][:g.k])
            y_eff, m_eff = data.y[r0:r0 + L].long(), mask_all[r0:r0 + L]
        self.y_eff, self.mask_eff = y_eff.to(dev), m_eff.to(dev)
        self.train_count_global = int(mask_all.sum())
        self.local_train_rows = int(m_eff.sum())
        per = classes // g.q
        self.cls_lo = g.j * per
        self.cls_hi = classes if g.j == g.q - 1 else (g.j + 1) * per

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
    """gcn_distr_3d.py:1054-1141."""
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
