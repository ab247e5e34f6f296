"""Per-category wall-clock accumulators with the reference's category names and report format
(gcn_distr.py:42-94, 613-637; gcn_distr_15d.py:67-99, 662-672; gcn_distr_2d.py:109-131, 1324-1344).

With `--timing=True` every bracketed region is fenced by a device synchronisation, as the 1.5D/2D/3D
reference scripts do, which serialises communication and compute; with timing off the brackets cost
nothing and the schedules overlap.

Beyond the reference: every collective is also booked under a name of its own with the bytes it moves over the
links (`comm`, `traffic`), and `event_mode` replaces the host fences by CUDA events recorded on the launching
stream, so that one instrumented epoch gives milliseconds and bytes per collective without stopping the device
(the benchmark's "collectives" field).
"""
import time
from contextlib import contextmanager


def all_reduce_bytes(nbytes, members):
    """Bytes one rank sends (and receives) in a bandwidth-optimal all-reduce of an nbytes buffer."""
    return 0 if members <= 1 else int(2 * nbytes * (members - 1) / members)


def all_gather_bytes(chunk_bytes, members):
    """Bytes one rank receives in an all-gather of chunk_bytes per member."""
    return int(chunk_bytes * max(members - 1, 0))

CATEGORIES_1D = ("comm_time", "comp_time", "scomp_time", "dcomp_time", "bcast_comm_time", "barrier_time",
                 "barrier_subset_time", "op1_comm_time", "op2_comm_time")
CATEGORIES_15D = ("comm_time", "comp_time", "scomp_time", "dcomp_time", "bcast_comm_time", "bcast_words",
                  "reduce_comm_time", "op_comm_time", "barrier_time")
CATEGORIES_2D = ("comm_time", "comp_time", "summa_sparse_comp", "summa_sparse_bcast1", "summa_sparse_bcast1_words",
                 "summa_sparse_bcast2", "summa_sparse_bcast2_fwd", "summa_sparse_bcast2_bwd",
                 "summa_sparse_bcast2_words", "summa_comp", "summa_bcast1", "summa_bcast2", "summa_loc_bcast",
                 "transpose_time", "grad_weight_time", "loss_calc_time", "summa_sparse_time", "summa_time",
                 "summa_loc_time")
CATEGORIES_3D = ("comm_time", "comp_time", "summa_sparse_comp", "summa_sparse_bcast1", "summa_sparse_bcast1_words",
                 "summa_sparse_bcast2", "summa_sparse_reduce", "summa_sparse_bcast2_words", "summa_comp",
                 "summa_bcast1", "summa_bcast2", "summa_reduce", "summa_loc_bcast", "transpose_time",
                 "loss_calc_time")


class Timers:
    def __init__(self, categories, enabled=False, sync=None):
        self.categories = tuple(categories)
        self.enabled = bool(enabled)
        self.sync = sync if sync is not None else (lambda: None)
        self.runs = {}
        self.run = 0
        self.event_mode = False          # with `enabled`: time regions by CUDA events instead of fenced wall clock
        self.make_event = None           # () -> an object with .record() and .elapsed_time(other), set by the caller
        self._pending = []               # (names, start event, stop event) not yet added up
        self.links = {}                  # collective name -> [calls, bytes, milliseconds]
        self.start_run(0)

    def start_run(self, run):
        self.run = run
        self.runs[run] = {c: 0.0 for c in self.categories}
        self.runs[run]["total_time"] = 0.0

    def add(self, category, value):
        if category in self.runs[self.run]:
            self.runs[self.run][category] += value

    def count(self, category, value):
        """Counters (e.g. words broadcast) accumulate whether or not timing is on."""
        self.add(category, value)

    def traffic(self, name, nbytes):
        """Book one collective call under `name`: nbytes = what this rank moves over the links for it."""
        rec = self.links.setdefault(name, [0, 0, 0.0])
        rec[0] += 1
        rec[1] += int(nbytes)

    @contextmanager
    def comm(self, name, nbytes, *categories):
        """A blocking collective: booked under `name`, timed (when timing is on) under `categories` and `name`."""
        self.traffic(name, nbytes)
        with self.region(*categories, "link:" + name):
            yield

    def use_events(self, make_event):
        """Time regions with device events from now on: no host fences, the stream keeps running."""
        self.event_mode, self.make_event, self.enabled = True, make_event, True

    def flush_events(self):
        """Add up the recorded regions; the caller has synchronised the device."""
        for names, e0, e1 in self._pending:
            ms = e0.elapsed_time(e1)
            for c in names:
                if c.startswith("link:"):
                    self.links.setdefault(c[5:], [0, 0, 0.0])[2] += ms
                else:
                    self.add(c, ms / 1e3)
        self._pending = []

    @contextmanager
    def region(self, *categories):
        if not self.enabled:
            yield
            return
        if self.event_mode:
            e0, e1 = self.make_event(), self.make_event()
            e0.record()
            try:
                yield
            finally:
                e1.record()
                self._pending.append((categories, e0, e1))
            return
        self.sync()
        t0 = time.time()
        try:
            yield
        finally:
            self.sync()
            dt = time.time() - t0
            for c in categories:
                if c.startswith("link:"):
                    self.links.setdefault(c[5:], [0, 0, 0.0])[2] += dt * 1e3
                else:
                    self.add(c, dt)

    @contextmanager
    def paused(self):
        was, self.enabled = self.enabled, False
        try:
            yield
        finally:
            self.enabled = was

    def report(self, rank, run, total_label="total_time", printer=print):
        rec = self.runs[run]
        printer(f"rank: {rank} {total_label}: {rec['total_time']}")
        for c in self.categories:
            printer(f"rank: {rank} {c}: {rec[c]}")
