"""1D (block-row) and 1.5D (block-row with replication factor c) full-batch GCN training.

Host-side mirror of the reference's `gcn_distr.py` and `gcn_distr_15d.py`: same function names and
argument meaning (`broad_func`, `GCNFunc`, `outer_product2`, `train`, `run`), same block schedule and
collectives, same loss and update rule.  What differs is underneath: every local computation is a
kernel of the native library on cached int32 CSR blocks, activations are fused into the dense product,
the backward of the activation is closed-form, and the broadcast of block k+1 runs on NCCL's stream while
block k is being multiplied.  With replication = 1 the 1.5D schedule IS the 1D one (P stages, source i
at stage i), so one implementation serves both scripts.
"""
import math
import statistics
import time

import torch
import torch.distributed as dist
import torch.nn.functional as F

from . import partition
from .backend import ACT_LOG_SOFTMAX, ACT_NONE, ACT_RELU


def ops_pad_ld(f):
    """Padded row length of an f-wide matrix (the rule of ops.pad_ld, restated so that this module does not need the
    native library to be importable)."""
    return (f + 3) // 4 * 4 if f <= 64 else (f + 31) // 32 * 32
from .timing import CATEGORIES_15D, CATEGORIES_1D, Timers, all_gather_bytes, all_reduce_bytes


class Data:
    """Attribute bag with the two fields the training loop reads: `y` (int64 labels) and `train_mask`."""

    def __init__(self, **kw):
        self.__dict__.update(kw)

    def to(self, device):
        for k, v in list(self.__dict__.items()):
            if torch.is_tensor(v):
                self.__dict__[k] = v.to(device)
        return self


class Runtime:
    """Per-process settings: what the reference keeps in module globals (gcn_distr.py:53-64)."""

    def __init__(self, backend, activations=True, normalization=True, replication=1, timing=False, overlap=True,
                 categories=None, order="reference", stage_groups=-1, collective="all_gather", prefetch_features=False,
                 directed=False):
        if order not in ("reference", "min_width"):
            raise ValueError("order must be 'reference' or 'min_width'")
        if collective not in ("all_gather", "broadcast"):
            raise ValueError("collective must be 'all_gather' or 'broadcast'")
        # how the H blocks of a 1D sparse product travel: "broadcast" = one broadcast per source rank, as the
        # reference issues them; "all_gather" = the same bytes in one collective per launch group
        self.collective = collective
        self.order = order
        # launch groups per sparse product: 0 = one per stage, as the reference; -1 = automatic (see Model)
        self.stage_groups = stage_groups
        self.backend = backend
        self.activations = bool(activations)
        self.normalization = bool(normalization)
        self.replication = int(replication)
        self.overlap = bool(overlap)
        # 1D all-gather schedule only: the vertex features never change between epochs (the reference reads the same
        # `inputs_loc` every epoch, gcn_distr.py:595-601), so the all-gather of layer 1 for epoch k+1 depends on
        # nothing epoch k computes.  With this on it is issued, on a communicator of its own, as soon as epoch k's
        # layer-1 multiply is queued and travels under the rest of epoch k; the same bytes move every epoch.
        # `next_features` = (tensor, event or None): the features of the NEXT epoch when they differ from the current
        # ones (a loader that refills a second buffer) and the event that marks them ready.
        self.prefetch_features = bool(prefetch_features)
        self.prefetch_group = None
        # The reference multiplies by the forward pass's blocks again in the backward pass: exact when the
        # adjacency matrix is symmetric (gcn_distr.py:326, gcn_distr_2d.py:683 "only true for undirected graphs").
        # `directed` partitions the transposed operator as well and multiplies the backward pass by that: twice
        # the adjacency storage, the true gradients for a graph whose edge list is not symmetric.
        self.directed = bool(directed)
        self.next_features = None
        self.layer1_input = None
        cats = categories or (CATEGORIES_15D if replication > 1 else CATEGORIES_1D)
        self.timers = Timers(cats, timing, getattr(backend, "synchronize", None))


def act_name(func):
    if func is F.relu or func == ACT_RELU:
        return ACT_RELU
    if func is F.log_softmax or func == ACT_LOG_SOFTMAX:
        return ACT_LOG_SOFTMAX
    return ACT_NONE


# ------------------------------------------------------------------------------------------ schedule
class StageGroup:
    """Consecutive stages of one rank multiplied in ONE launch: their H blocks are received into adjacent row
    ranges of one buffer and the adjacency blocks are fused column-wise into one CSR block."""

    def __init__(self, sources, block, rows):
        self.sources, self.block, self.rows = sources, block, rows     # sources: [(source rank, rows of its H block)]


class StagePlan:
    """The stages `rank` walks through (gcn_distr_15d.py:194-208), cut into `groups` launch groups.

    groups = number of stages reproduces the reference's granularity (one broadcast, one multiply per stage).
    Fewer groups trade pipeline depth for larger multiplies: on a 233K-vertex graph split 8 ways one launch per
    stage spends most of its time on per-launch and per-row-segment overheads (6.5 ms against 4.1 ms for the same
    nonzeros in one launch at width 602, 1.29 ms against 0.39 ms at width 16), while the broadcasts it could hide
    take 0.7 ms in total.  `Model` passes one group unless told otherwise; two keep the broadcast of the second half
    behind the multiply of the first."""

    def __init__(self, backend, blocks, rank, size, replication, groups=1):
        stages = partition.stages_15d(rank, size, replication)
        self.n_loc = blocks[0].n_rows
        n_groups = max(1, min(len(stages), groups if groups and groups > 0 else len(stages)))
        bounds = [round(i * len(stages) / n_groups) for i in range(n_groups + 1)]
        self.groups = []
        for a, b in zip(bounds[:-1], bounds[1:]):
            part = stages[a:b]
            fused = partition.fuse_columns([blocks[bid] for _, bid in part])
            sources = [(q, blocks[bid].n_cols) for q, bid in part]
            self.groups.append(StageGroup(sources, backend.make_block(fused), fused.n_cols))
        self.max_rows = max(g.rows for g in self.groups) if self.groups else 0


class GatherGroup:
    def __init__(self, lo, rows, block):
        self.lo, self.rows, self.block = lo, rows, block      # rows [lo, lo + rows) of every rank's H block


class GatherPlan:
    """1D only: the P broadcasts of one sparse product taken as what they add up to, an all-gather.

    Every rank's H block is cut into the same `groups` row ranges; launch group g all-gathers range g of every
    block into one buffer (rank i's rows at i * rows_g) and multiplies it by the columns of this rank's block row
    that fall in those ranges, fused into one CSR block with the columns renumbered to buffer positions.  The last
    block may be shorter than the others: its missing rows are sent as padding that no column refers to.
    One NCCL call moves what P broadcast calls moved; at 8 GPUs and width 602 the eight 70 MB broadcasts cost
    about 2.5 ms per product, the all-gather of the same bytes well under 1 ms."""

    def __init__(self, backend, blocks, rank, size, n_per_proc, groups=1):
        self.n_loc = blocks[0].n_rows
        self.size = size
        # feature prefetch (Runtime.prefetch_features): {(data pointer, width): [(buffer, work)]} posted for the next
        # epoch, two buffer sets used in turn
        self.prefetched, self.prefetch_bufs, self.flip = {}, {}, 0
        n_groups = max(1, min(groups if groups and groups > 0 else 1, n_per_proc))
        bounds = [round(g * n_per_proc / n_groups) for g in range(n_groups + 1)]
        self.groups = []
        for lo, hi in zip(bounds[:-1], bounds[1:]):
            rows = hi - lo
            parts = []
            for i, b in enumerate(blocks):
                sel = (b.cols >= lo) & (b.cols < hi)
                parts.append(partition.Block(b.rows[sel], b.cols[sel] - lo + i * rows, b.vals[sel], b.n_rows, size * rows))
            r = torch.cat([p.rows for p in parts])
            c = torch.cat([p.cols for p in parts])
            v = torch.cat([p.vals for p in parts])
            order = torch.argsort(r * (size * rows) + c)
            # the diagonal factors of the fused block: this rank's row factor, and per buffer position the column
            # factor of the vertex that lands there (padding positions, which no column refers to, get 0)
            row_scale = col_scale = None
            if all(b.row_scale is not None and b.col_scale is not None for b in blocks):
                row_scale = blocks[0].row_scale
                col_scale = torch.zeros(size * rows, dtype=torch.float32, device=row_scale.device)
                for i, b in enumerate(blocks):
                    piece = b.col_scale[lo:hi]
                    col_scale[i * rows:i * rows + piece.numel()] = piece
            fused = partition.Block(r[order], c[order], v[order], self.n_loc, size * rows, row_scale, col_scale)
            self.groups.append(GatherGroup(lo, rows, backend.make_block(fused)))


def _gather_func(rt, plan, inputs, rank, size, group):
    be = rt.backend
    f = inputs.size(1)
    comm = size > 1 and dist.is_initialized()
    z = be.empty(plan.n_loc, f)
    bufs = [None, None]
    ld = inputs.stride(0) if inputs.size(0) > 1 else f                  # floats per row on the wire

    def send_rows(src, g):
        have = max(0, min(src.size(0), g.lo + g.rows) - g.lo)          # the last block may end inside the range
        if have == g.rows:
            return src[g.lo:g.lo + g.rows]
        send = be.zeros(g.rows, f)
        if have > 0:
            be.wire(send[:have]).copy_(be.wire(src[g.lo:g.lo + have]))
        return send

    def post(gi):
        g = plan.groups[gi]
        send = send_rows(inputs, g)
        if not comm:
            return send, None
        if bufs[gi % 2] is None:
            bufs[gi % 2] = be.empty(size * max(gg.rows for gg in plan.groups), f)
        recv = bufs[gi % 2][:size * g.rows]
        rt.timers.count("bcast_words", size * g.rows * f)
        rt.timers.traffic("h_all_gather", all_gather_bytes(g.rows * ld * 4, size))
        work = dist.all_gather_into_tensor(be.wire(recv), be.wire(send), group=group, async_op=True)
        return recv, work

    serial = rt.timers.enabled or not rt.overlap
    layer1 = comm and rt.prefetch_features and rt.layer1_input is not None and inputs.data_ptr() == rt.layer1_input
    ready = plan.prefetched.pop((inputs.data_ptr(), f), None) if layer1 else None
    pending = None
    for gi, g in enumerate(plan.groups):
        if ready is not None:
            tensor, work = ready[gi]
            if work is not None:
                work.wait()
        elif serial:
            with rt.timers.region("comm_time", "bcast_comm_time", "link:h_all_gather"):
                tensor, work = post(gi)
                if work is not None:
                    work.wait()
        else:
            tensor, work = pending if pending is not None else post(gi)
            pending = post(gi + 1) if gi + 1 < len(plan.groups) else None
            if work is not None:
                work.wait()
        with rt.timers.region("comp_time", "scomp_time"):
            be.spmm(g.block, tensor, z, 0.0 if gi == 0 else 1.0)
    if layer1 and not rt.timers.enabled:
        # next epoch's gather of the features, into the buffer set this epoch did not read
        nxt, event = rt.next_features if rt.next_features is not None else (inputs, None)
        nxt = be.as_matrix(nxt)
        if event is not None:
            torch.cuda.current_stream().wait_event(event)
        plan.flip ^= 1
        posted = []
        for gi, g in enumerate(plan.groups):
            key = (plan.flip, gi)
            if key not in plan.prefetch_bufs:
                plan.prefetch_bufs[key] = be.empty(size * g.rows, f)
            recv = plan.prefetch_bufs[key]
            rt.timers.count("bcast_words", size * g.rows * f)
            rt.timers.traffic("h_all_gather", all_gather_bytes(g.rows * ld * 4, size))
            posted.append((recv, dist.all_gather_into_tensor(be.wire(recv), be.wire(send_rows(nxt, g)),
                                                             group=rt.prefetch_group, async_op=True)))
        plan.prefetched = {(nxt.data_ptr(), f): posted}
    return z


def broad_func(rt, node_count, am_partitions, inputs, rank, size, row_groups, col_groups, group):
    if isinstance(am_partitions, GatherPlan):
        return _gather_func(rt, am_partitions, rt.backend.as_matrix(inputs), rank, size, group)
    return _broadcast_func(rt, node_count, am_partitions, inputs, rank, size, row_groups, col_groups, group)


def _broadcast_func(rt, node_count, am_partitions, inputs, rank, size, row_groups, col_groups, group):
    """Z_r = sum over this rank's stages of A_blk[stage] . H_stage, then (1.5D) an all-reduce of Z_r over the
    c replicas of the block row.  gcn_distr.py:203-246, gcn_distr_15d.py:173-245.  `am_partitions` is the
    rank's StagePlan.

    Every stage broadcasts one block of H inside the rank's column communicator; the stages of a launch group
    land in one buffer and are multiplied by the group's fused CSR block.  Two buffers alternate: the broadcasts
    of group k+1 are issued (async) before the multiply of group k is queued, so NCCL moves the next blocks while
    the SMs work on the current ones."""
    be, c = rt.backend, rt.replication
    plan = am_partitions
    inputs = be.as_matrix(inputs)
    f = inputs.size(1)
    rank_c, rank_col = rank // c, rank % c
    col_group = col_groups[rank_col] if c > 1 else group
    row_group = row_groups[rank_c] if c > 1 else None
    comm = size > 1 and dist.is_initialized()
    z = be.empty(plan.n_loc, f)
    if not plan.groups:
        be.wire(z).zero_()
    bufs = [None, None]

    def post(gi):
        g = plan.groups[gi]
        if len(g.sources) == 1 and g.sources[0][0] == rank:
            tensor, pieces = inputs, [(inputs, rank)]
        else:
            if bufs[gi % 2] is None:
                bufs[gi % 2] = be.empty(plan.max_rows, f)
            tensor, pieces, off = bufs[gi % 2][:g.rows], [], 0
            for q, rows in g.sources:
                piece = tensor[off:off + rows]
                if q == rank:
                    be.wire(piece).copy_(be.wire(inputs))       # this rank's own block takes its place in the buffer
                pieces.append((piece, q))
                off += rows
        works = []
        for piece, q in pieces:
            rt.timers.count("bcast_words", piece.size(0) * f)
            if comm:
                rt.timers.traffic("h_broadcast", be.wire(piece).numel() * 4)
                works.append(dist.broadcast(be.wire(piece), src=q, group=col_group, async_op=True))
        return tensor, works

    serial = rt.timers.enabled or not rt.overlap
    pending = None
    for gi, g in enumerate(plan.groups):
        if serial:
            with rt.timers.region("comm_time", "bcast_comm_time", "link:h_broadcast"):
                tensor, works = post(gi)
                for w in works:
                    w.wait()
        else:
            tensor, works = pending if pending is not None else post(gi)
            pending = post(gi + 1) if gi + 1 < len(plan.groups) else None
            for w in works:
                w.wait()                         # stream-side wait: the host runs ahead
        with rt.timers.region("comp_time", "scomp_time"):
            be.spmm(g.block, tensor, z, 0.0 if gi == 0 else 1.0)
    if c > 1 and comm:
        with rt.timers.comm("z_replica_all_reduce", all_reduce_bytes(be.wire(z).numel() * 4, c), "comm_time",
                            "reduce_comm_time"):
            dist.all_reduce(be.wire(z), op=dist.ReduceOp.SUM, group=row_group)
    return z


def outer_product2(rt, inputs, ag, rank, size, group):
    """grad_W = H^T . (A G), summed over the block rows (gcn_distr.py:178-201)."""
    be = rt.backend
    with rt.timers.region("comp_time", "dcomp_time"):
        grad_weight = be.mm_tn(be.as_matrix(inputs), ag)
    if size > 1 and dist.is_initialized():
        members = size // rt.replication
        with rt.timers.comm("grad_w_all_reduce", all_reduce_bytes(grad_weight.numel() * 4, members), "comm_time",
                            "op2_comm_time", "op_comm_time"):
            dist.all_reduce(grad_weight, op=dist.ReduceOp.SUM, group=group)
    return grad_weight


class GCNFunc(torch.autograd.Function):
    """One GCN layer: out = act((A . H) . W).  gcn_distr.py:248-339, gcn_distr_15d.py:247-345.

    With `rt.order == "min_width"` (off by default) the sparse product always runs at the narrower of the two
    widths: forward takes A . (H . W) when the layer narrows, and a widening layer's backward takes
    grad_H = A . (dZ . W^T) and grad_W = (A . H)^T . dZ with A . H kept from the forward pass.  The results are the
    reference's up to the order of summation; the second identity needs A = A^T, which the reference's own
    backward already assumes by multiplying with the forward blocks (gcn_distr.py:326)."""

    @staticmethod
    def forward(ctx, inputs, weight, adj_matrix, am_partitions, rank, size, group, row_groups, col_groups, func, rt):
        be = rt.backend
        act = act_name(func) if rt.activations else ACT_NONE
        w = weight.detach()
        narrow = rt.order == "min_width" and w.size(1) < w.size(0)
        widen = rt.order == "min_width" and w.size(1) > w.size(0)
        agg = None
        if narrow:
            with rt.timers.region("comp_time", "dcomp_time"):
                hw = be.mm(be.as_matrix(inputs), w, ACT_NONE)
            z = broad_func(rt, None, am_partitions, hw, rank, size, row_groups, col_groups, group)
            with rt.timers.region("comp_time", "dcomp_time"):
                out = be.act(z, act)
        else:
            z = broad_func(rt, None, am_partitions, inputs, rank, size, row_groups, col_groups, group)
            with rt.timers.region("comp_time", "dcomp_time"):
                out = be.mm(z, w, act)
            if widen:
                agg = z
        ctx.save_for_backward(inputs, weight, out)
        ctx.agg = agg
        # backward multiplies by the transposed operator's plan when the model built one (directed graphs)
        ctx.args = (getattr(am_partitions, "backward_plan", None) or am_partitions, rank, size, group, row_groups,
                    col_groups, act, rt)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        inputs, weight, out = ctx.saved_tensors
        am_partitions, rank, size, group, row_groups, col_groups, act, rt = ctx.args
        be = rt.backend
        w = weight.detach()
        reduce_group = col_groups[rank % rt.replication] if rt.replication > 1 else group
        # sigma'(Z) * G in closed form from the activation output (the reference re-runs the activation
        # under autograd: gcn_distr.py:312-322)
        dz = be.act_bwd(out, be.as_matrix(grad_output), act)
        if ctx.agg is not None:
            grad_input = None
            if ctx.needs_input_grad[0]:
                with rt.timers.region("comp_time", "dcomp_time"):
                    dzw = be.mm_nt(dz, w)
                grad_input = broad_func(rt, None, am_partitions, dzw, rank, size, row_groups, col_groups, group)
            grad_weight = outer_product2(rt, ctx.agg, dz, rank, size, reduce_group)
            return grad_input, grad_weight, None, None, None, None, None, None, None, None, None
        ag = broad_func(rt, None, am_partitions, dz, rank, size, row_groups, col_groups, group)
        grad_input = None
        if ctx.needs_input_grad[0]:
            with rt.timers.region("comp_time", "dcomp_time"):
                grad_input = be.mm_nt(ag, w)
        grad_weight = outer_product2(rt, inputs, ag, rank, size, reduce_group)
        return grad_input, grad_weight, None, None, None, None, None, None, None, None, None


class MaskedNLL(torch.autograd.Function):
    """mean over the masked rows of -outputs[i, y_i] (F.nll_loss(outputs[mask], y[mask]), gcn_distr.py:356),
    loss and gradient from one fused kernel."""

    @staticmethod
    def forward(ctx, outputs, y, mask, count, rt, cls_lo, cls_hi, denom):
        loss, grad = rt.backend.nll(rt.backend.as_matrix(outputs), y, mask, denom, cls_lo, cls_hi)
        ctx.grad = grad
        ctx.wire = rt.backend.wire
        return loss

    @staticmethod
    def backward(ctx, g):
        grad = ctx.grad
        ctx.wire(grad).mul_(g)
        return grad, None, None, None, None, None, None, None


class Model:
    """What `run()` builds once per process: cached device blocks, this rank's features, labels and mask."""

    def __init__(self, rt, rank, size, inputs, adj_matrix, data, features, classes, group=None, row_groups=None,
                 col_groups=None):
        be, c = rt.backend, rt.replication
        self.rt, self.rank, self.size, self.features, self.classes = rt, rank, size, features, classes
        self.group, self.row_groups, self.col_groups = group, row_groups, col_groups
        node_count = inputs.size(0)
        self.node_count = node_count
        # degrees: every rank counts 1/P of the edge list, one all-reduce (all ranks hold the same list and are here)
        everyone = group if (group is not None and size % c == 0) else None
        inputs_loc, blocks = partition.oned_partition(rank, size, inputs, adj_matrix, rt.normalization, c,
                                                      degree_group=everyone)
        self.inputs_loc = be.as_matrix(inputs_loc)
        n_per_proc = int(math.ceil(float(node_count) / (size / c)))
        # Automatic launch groups.  More groups put the communication of group g+1 under the multiply of group g, but
        # every group is a block of its own: its dense core is smaller or gone, and each launch costs the same however
        # little it does.  So: ONE group while a stage's H block is small (233K-vertex benchmark graph, 70-283 MB per
        # stage: 2 ranks 9.72 ms with one group against 10.06 with two; 8 ranks 6.8 against 7.6), and pipelined
        # groups once a stage moves half a gigabyte or more, where the gathers are the larger cost (1.33 B-edge graph,
        # 1D: 4 ranks 95.0 -> 89.8 ms, 8 ranks 57.8 -> 48.3 ms with four groups; 14 M-vertex graph, 1.5D c = 2, 8 ranks:
        # 42.5 -> 39.3 ms with one group per stage).  Every rank computes the same figure from global sizes.
        if rt.stage_groups >= 0:
            groups = rt.stage_groups
        elif size > 1 and n_per_proc * ops_pad_ld(int(inputs.size(1))) * 4 >= (512 << 20):
            groups = 4 if (c == 1 and rt.collective == "all_gather") else 0
        else:
            groups = 1
        self.launch_groups = groups
        def make_plan(blks):
            if c == 1 and size > 1 and rt.collective == "all_gather":
                return GatherPlan(be, blks, rank, size, n_per_proc, groups)
            return StagePlan(be, blks, rank, size, c, groups)

        self.am_pbyp = make_plan(blocks)
        if isinstance(self.am_pbyp, GatherPlan) and rt.prefetch_features and dist.is_initialized() \
                and rt.prefetch_group is None:
            # a communicator of its own: the prefetch must not queue in front of the epoch's other collectives
            rt.prefetch_group = dist.new_group(list(range(size)))
        if rt.directed:
            _, blocks_t = partition.oned_partition(rank, size, inputs, adj_matrix, rt.normalization, c,
                                                   degree_group=everyone, transposed=True)
            self.am_pbyp.backward_plan = make_plan(blocks_t)
        rank_c = rank // c
        lo, hi = rank_c * n_per_proc, min(node_count, (rank_c + 1) * n_per_proc)
        dev = self.inputs_loc.device
        self.rank_train_mask = data.train_mask[lo:hi].bool().to(dev)
        self.datay_rank = data.y[lo:hi].long().to(dev)
        self.train_count = int(self.rank_train_mask.sum())

    def init_weights(self, mid_layer, capturable=False):
        """torch.manual_seed(0); rand on the CPU, then moved (gcn_distr.py:550-560).  `capturable` keeps Adam's
        step count on the device so that an epoch can be recorded into a CUDA graph (see `capture`)."""
        torch.manual_seed(0)
        dev = self.inputs_loc.device
        w1 = torch.rand(self.features, mid_layer, requires_grad=True).to(dev)
        w2 = torch.rand(mid_layer, self.classes, requires_grad=True).to(dev)
        self.weight1 = torch.nn.Parameter(w1.detach())
        self.weight2 = torch.nn.Parameter(w2.detach())
        self.optimizer = torch.optim.Adam([self.weight1, self.weight2], lr=0.01, capturable=bool(capturable))
        self._graph = self._graph_outputs = None
        return self.weight1, self.weight2

    def _train_eager(self):
        return train(self.inputs_loc, self.weight1, self.weight2, None, self.am_pbyp, self.optimizer, self,
                     self.rank, self.size, self.group, self.row_groups, self.col_groups, self.rt)

    def train(self):
        """One epoch; returns this rank's output rows, detached.  (A caller that kept attached outputs of an eager
        epoch would keep that epoch's autograd graph alive, and with it the weights' gradient accumulators, which
        remember the stream they were created under -- a later `capture()` on its own stream then fails.)"""
        if getattr(self, "_graph", None) is not None:
            self._graph.replay()
            return self._graph_outputs
        return self._train_eager().detach()

    def capture(self):
        """Record one whole epoch (both layers, loss, backward, collectives, Adam) into a CUDA graph; `train()`
        replays it from then on (single process only).  An epoch is ~30 launches of this library plus the
        optimizer's; replaying them as one graph takes the host out of the loop.  Call after at
        least one eager epoch (communicators, Adam state and block caches must exist) with weights created by
        `init_weights(..., capturable=True)`; the features, labels and mask are read from the tensors the model
        holds at capture time, so new data has to be copied INTO them.  Capturing does not execute an epoch."""
        if self.rt.timers.enabled:
            raise RuntimeError("cagnet_b200: an epoch cannot be captured with --timing=True (it synchronises)")
        if self.size > 1 and dist.is_initialized():
            # recording the NCCL calls of an epoch did not return on 2 GPUs with this torch / NCCL pair
            raise RuntimeError("cagnet_b200: epoch capture is single-process only; multi-rank epochs run eagerly")
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, capture_error_mode="thread_local"):
            outputs = self._train_eager().detach()
        self._graph, self._graph_outputs = graph, outputs
        return graph


def train(inputs, weight1, weight2, adj_matrix, am_partitions, optimizer, model, rank, size, group, row_groups,
          col_groups, rt):
    """One epoch: two layers, the rank-local mean NLL over its own train rows, backward, Adam step.
    gcn_distr.py:341-366.  `model` supplies this rank's label / mask slices and its train-row count."""
    rt.layer1_input = inputs.data_ptr()       # what the feature prefetch recognises the first layer's multiply by
    outputs = GCNFunc.apply(inputs, weight1, adj_matrix, am_partitions, rank, size, group, row_groups, col_groups,
                            F.relu, rt)
    rt.layer1_input = None
    outputs = GCNFunc.apply(outputs, weight2, adj_matrix, am_partitions, rank, size, group, row_groups, col_groups,
                            F.log_softmax, rt)
    optimizer.zero_grad()
    if model.train_count > 0:
        loss = MaskedNLL.apply(outputs, model.datay_rank, model.rank_train_mask, model.train_count, rt, 0, None,
                               model.train_count)
        loss.backward()
        model.last_loss = loss.detach()
    else:
        # no train rows here: a zero gradient still has to flow so that this rank joins the collectives of
        # the backward pass (the reference's "fake loss", gcn_distr.py:359-362)
        outputs.backward(rt.backend.zeros(outputs.size(0), outputs.size(1)))
        model.last_loss = torch.zeros((), device=outputs.device)
    optimizer.step()
    return outputs


def make_groups(rank, size, replication):
    """All-ranks group plus the 1.5D row / column communicators; every rank creates every group, in the
    same order (gcn_distr.py:532, gcn_distr_15d.py:398-419)."""
    if not dist.is_initialized() or size == 1:
        return None, None, None
    group = dist.new_group(list(range(size)))
    if replication == 1:
        return group, None, None
    rows, cols = partition.proc_groups_15d(size, replication)
    row_groups = [dist.new_group(r) for r in rows]
    col_groups = [dist.new_group(c) for c in cols]
    return group, row_groups, col_groups


def run(rank, size, inputs, adj_matrix, data, features, classes, rt, epochs, mid_layer, run_count, accuracy=False,
        printer=print):
    """Partition, then `run_count` runs of: reseed weights, one untimed epoch, `epochs - 1` timed epochs; report
    the median run by rank-0 wall time with its per-category breakdown.  gcn_distr.py:524-669."""
    group, row_groups, col_groups = make_groups(rank, size, rt.replication)
    if rank // rt.replication >= size // rt.replication:
        return None
    model = Model(rt, rank, size, inputs, adj_matrix, data, features, classes, group, row_groups, col_groups)
    printer(f"rank: {rank} adj_matrix_loc.size: torch.Size([{model.node_count}, {model.inputs_loc.size(0)}])")
    printer(f"rank: {rank} inputs.size: {tuple(inputs.size())}")
    timers = rt.timers
    outputs = None
    comm = group is not None

    def sync():
        if hasattr(rt.backend, "synchronize"):
            rt.backend.synchronize()

    for i in range(run_count):
        timers.start_run(i)
        model.init_weights(mid_layer)
        if comm:
            dist.barrier(group)
        with timers.paused():                       # the first epoch is not timed
            outputs = model.train()
        if comm:
            dist.barrier(group)
        sync()
        tstart = time.time()
        printer(f"Starting training... rank {rank} run {i}")
        for epoch in range(1, epochs):
            outputs = model.train()
            printer("Epoch: {:03d}".format(epoch))
        sync()
        timers.runs[i]["total_time"] = time.time() - tstart

    if comm:
        dist.barrier(group)
    totals = [timers.runs[i]["total_time"] for i in range(run_count)]
    median_idx = totals.index(statistics.median_low(totals))
    if comm:
        idx = torch.tensor([median_idx], device=model.inputs_loc.device)
        dist.broadcast(idx, src=0, group=group)
        median_idx = int(idx.item())
    if rank == 0:
        printer(f"total_times_r0: {totals}")
    printer(f"rank: {rank} median_run: {median_idx}")
    timers.report(rank, median_idx, printer=printer)
    printer(f"rank: {rank} {outputs}")

    if accuracy:
        gathered = gather_outputs(model, outputs)
        accs = test(gathered, data)
        printer("Epoch: {:03d}, Train: {:.4f}, Val: {:.4f}, Test: {:.4f}".format(900, accs[0], accs[1], accs[2]))
    model.outputs = outputs
    return model


def gather_outputs(model, outputs):
    """All block rows of the final activations on every rank (gcn_distr.py:641-659)."""
    rt, size, rank = model.rt, model.size, model.rank
    c = rt.replication
    rows_of = size // c
    n, classes = model.node_count, model.classes
    n_per_proc = int(math.ceil(float(n) / (size / c)))
    dense = outputs.detach().contiguous()
    if model.group is None:
        return dense
    if dense.size(0) != n_per_proc:
        pad = torch.zeros(n_per_proc - dense.size(0), classes, device=dense.device)
        dense = torch.cat([dense, pad], dim=0)
    parts = [torch.zeros_like(dense) for _ in range(rows_of)]
    dist.all_gather(parts, dense, group=model.col_groups[rank % c] if c > 1 else model.group)
    return torch.cat(parts, dim=0)[:n]


def test(outputs, data):
    """Train / validation / test accuracy from gathered activations (gcn_distr.py:368-379)."""
    accs = []
    for name in ("train_mask", "val_mask", "test_mask"):
        mask = getattr(data, name, None)
        if mask is None:
            accs.append(0)
            continue
        mask = mask.bool().to(outputs.device)
        pred = outputs[mask].max(1)[1]
        accs.append(pred.eq(data.y.to(outputs.device)[mask]).sum().item() / max(int(mask.sum().item()), 1))
    return accs
