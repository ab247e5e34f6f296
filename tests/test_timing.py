"""Timing accumulators: the reference's category names, its report format, pause for the untimed first epoch."""
import time

from cagnet_b200.timing import CATEGORIES_15D, CATEGORIES_1D, CATEGORIES_2D, Timers


def test_regions_accumulate_only_when_enabled():
    syncs = []
    t = Timers(CATEGORIES_1D, enabled=True, sync=lambda: syncs.append(1))
    with t.region("comm_time", "bcast_comm_time"):
        time.sleep(0.01)
    assert t.runs[0]["comm_time"] >= 0.009 and t.runs[0]["bcast_comm_time"] == t.runs[0]["comm_time"]
    assert len(syncs) == 2                      # fenced before and after, as the 1.5D/2D/3D reference scripts do
    with t.paused():
        with t.region("comp_time"):
            time.sleep(0.005)
    assert t.runs[0]["comp_time"] == 0.0
    off = Timers(CATEGORIES_1D, enabled=False, sync=lambda: syncs.append(1))
    with off.region("comm_time"):
        pass
    assert off.runs[0]["comm_time"] == 0.0 and len(syncs) == 2


def test_report_lines_match_the_reference_format():
    t = Timers(CATEGORIES_15D, enabled=False)
    t.start_run(1)
    t.count("bcast_words", 1234)
    t.runs[1]["total_time"] = 2.5
    lines = []
    t.report(3, 1, printer=lines.append)
    assert lines[0] == "rank: 3 total_time: 2.5"
    assert "rank: 3 bcast_words: 1234.0" in lines
    assert [ln.split()[2].rstrip(":") for ln in lines[1:]] == list(CATEGORIES_15D)
    assert "summa_sparse_bcast1_words" in CATEGORIES_2D and "op2_comm_time" in CATEGORIES_1D


class _FakeEvent:
    """Stands in for a CUDA event: `record()` stamps a counter that advances by 2.5 "ms" per call."""
    clock = [0.0]

    def __init__(self):
        self.t = None

    def record(self):
        _FakeEvent.clock[0] += 2.5
        self.t = _FakeEvent.clock[0]

    def elapsed_time(self, other):
        return other.t - self.t


def test_collectives_are_booked_by_name_with_bytes_and_event_time():
    from cagnet_b200.timing import CATEGORIES_1D, Timers, all_gather_bytes, all_reduce_bytes
    assert all_reduce_bytes(1000, 1) == 0 and all_reduce_bytes(1000, 4) == 1500
    assert all_gather_bytes(1000, 8) == 7000 and all_gather_bytes(1000, 1) == 0
    t = Timers(CATEGORIES_1D, enabled=False)
    with t.comm("h_all_gather", 4096, "comm_time", "bcast_comm_time"):      # timing off: bytes and calls only
        pass
    t.traffic("h_all_gather", 1024)
    assert t.links["h_all_gather"] == [2, 5120, 0.0]
    assert t.runs[0]["comm_time"] == 0.0
    _FakeEvent.clock[0] = 0.0
    t.use_events(_FakeEvent)
    assert t.enabled and t.event_mode
    with t.comm("grad_w_all_reduce", 64, "comm_time", "op2_comm_time"):
        pass
    with t.region("comp_time", "scomp_time"):
        pass
    assert t.links["grad_w_all_reduce"] == [1, 64, 0.0]                      # nothing is added up before the flush
    t.flush_events()
    assert t.links["grad_w_all_reduce"] == [1, 64, 2.5]
    assert abs(t.runs[0]["comm_time"] - 2.5e-3) < 1e-12 and abs(t.runs[0]["scomp_time"] - 2.5e-3) < 1e-12
    assert t._pending == []
