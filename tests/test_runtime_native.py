"""Host-side C++ runtime: layouts, mailbox state machine, Lane scheduler, ECS seqlock channel,
CPU transport mailbox between processes, trace buffers. No GPU involved; failures are injected on
the host (a consumer that never answers, a closed mailbox)."""
import ctypes
import multiprocessing as mp
import os
import threading
import time

import numpy as np
import pytest

from crosspool_b200 import native
from crosspool_b200.native import runtime as rt


def test_abi_and_record_sizes():
    assert rt.lib().xr_abi_version() == native.EXPECTED_ABI
    assert rt.lib().xr_record_bytes(0) == 256  # InvocationRecord
    assert rt.lib().xr_record_bytes(1) == 256  # CompletionRecord


def test_slot_layouts_are_aligned_and_disjoint():
    f = rt.plan_ffn_slot(256, 1024, 3072)
    assert f.record_offset == 0 and f.input_offset % 256 == 0 and f.act_offset % 256 == 0
    assert f.act_offset >= f.input_offset + 256 * 1024 * 2
    assert f.total_bytes >= f.act_offset + 256 * 3072 * 2
    a = rt.plan_atn_slot(256, 1024, 4)
    assert a.output_offset >= 4 * 256 and a.output_stride >= 256 * 1024 * 2
    assert a.total_bytes == a.output_offset + 4 * a.output_stride
    with pytest.raises(ValueError):
        rt.plan_ffn_slot(2**40, 2**30, 8)


def test_mailbox_transition_table():
    ok = {(0, 1), (1, 2), (2, 3), (3, 4), (4, 1)}
    for a in range(6):
        for b in range(6):
            want = (a, b) in ok or b == rt.MBOX_CLOSED
            assert bool(rt.lib().xr_mailbox_transition_allowed(a, b)) == want, (a, b)


def test_scheduler_fifo_order_and_single_invocation_per_instance():
    s = rt.LaneScheduler(4, 2, rt.POLICY_FIFO)
    assert s.enqueue(2, 1) and s.enqueue(0, 1) and s.enqueue(3, 1)
    assert not s.enqueue(2, 2)  # already queued
    a = s.try_schedule()
    b = s.try_schedule()
    assert a[0] == 2 and b[0] == 0 and {a[1], b[1]} == {0, 1}
    assert s.try_schedule() is None  # both lanes busy
    assert s.active(2) == (a[1], a[2])
    assert not s.release(2, a[2] + 5)  # stale lease refused
    assert s.release(2, a[2])
    c = s.try_schedule()
    assert c[0] == 3 and c[1] == a[1]
    assert not s.enqueue(2, 1)  # sequence must advance past the completed one
    assert s.enqueue(2, 2)


def test_scheduler_slo_earliest_deadline_first_and_random_is_seeded():
    s = rt.LaneScheduler(3, 1, rt.POLICY_SLO)
    s.enqueue(0, 1, deadline=900)
    s.enqueue(1, 1, deadline=100)
    s.enqueue(2, 1, deadline=500)
    order = []
    for _ in range(3):
        i, lane, lease = s.try_schedule()
        order.append(i)
        s.release(i, lease)
    assert order == [1, 2, 0]
    # 32-bit microsecond stamps that wrap are ordered relative to one another; zero means "no deadline"
    w = rt.LaneScheduler(4, 1, rt.POLICY_SLO)
    w.enqueue(0, 1, deadline=0)
    w.enqueue(1, 1, deadline=50)               # wrapped: 150 us after instance 2's stamp
    w.enqueue(2, 1, deadline=2**32 - 100)
    w.enqueue(3, 1, deadline=2**32 - 5000)
    order = []
    for _ in range(4):
        i, lane, lease = w.try_schedule()
        order.append(i)
        w.release(i, lease)
    assert order == [3, 2, 1, 0]

    def run(seed):
        r = rt.LaneScheduler(8, 1, rt.POLICY_RANDOM, seed)
        for i in range(8):
            r.enqueue(i, 1)
        out = []
        for _ in range(8):
            i, lane, lease = r.try_schedule()
            out.append(i)
            r.release(i, lease)
        return out

    assert run(7) == run(7)
    assert sorted(run(7)) == list(range(8))
    assert run(7) != run(8) or run(7) != run(9)
    # the generator is the published SplitMix64
    assert rt.lib().xr_splitmix64(0) == 0xE220A8397B1DCDAF


def test_ecs_channel_roundtrip_between_handles():
    name = f"/xpool-test-ecs-{os.getpid()}"
    ch = rt.EcsChannel.create(name, devices=2, partitions=3, generation=5)
    try:
        ch.set_device(0, 0)
        ch.set_partition(1, device=0, group=0, rank=1, floor_bytes=1 << 20, reservation_bytes=8 << 20)
        other = rt.EcsChannel.attach(name)
        assert other.counts() == (2, 3, 5)
        assert other.partition(1)["reservation_bytes"] == 8 << 20
        ch.publish_command(1, 4, 123456)
        assert other.read_command(1) == (4, 123456)
        other.publish_demand(1, 4, 999, 10**9, 555)
        assert ch.read_demand(1) == (4, 999, 10**9, 555)
        other.publish_completion(1, 4, 777)
        assert ch.read_completion(1) == (4, 777)
        other.publish_report(0, 10, 20, 1)
        assert ch.read_report(0) == (10, 20, 1)
        other.close()
    finally:
        ch.close()
    with pytest.raises(OSError):
        rt.EcsChannel.attach(name)  # owner unlinked it


def test_ecs_seqlock_never_shows_a_torn_record():
    name = f"/xpool-test-seq-{os.getpid()}"
    ch = rt.EcsChannel.create(name, 1, 1)
    reader = rt.EcsChannel.attach(name)
    stop = threading.Event()

    def writer():
        i = 1
        while not stop.is_set():
            ch.publish_demand(0, i, i * 3, i * 7, i * 11)
            i += 1

    t = threading.Thread(target=writer)
    t.start()
    try:
        for _ in range(20000):
            a, b, c, d = reader.read_demand(0)
            assert (b, c, d) == (a * 3, a * 7, a * 11)
    finally:
        stop.set()
        t.join()
        reader.close()
        ch.close()


def _consumer(name, rows, row_bytes, n_requests, ready):
    mb = rt.CpuMailbox.attach(name, rows, row_bytes)
    mb.activate()
    ready.set()
    for _ in range(n_requests):
        rc, req = mb.take(5.0)
        assert rc == 0
        n, layer, mode, seq = req
        src = np.ctypeslib.as_array((ctypes.c_float * (n * row_bytes // 4)).from_address(mb.input_address))
        dst = np.ctypeslib.as_array((ctypes.c_float * (n * row_bytes // 4)).from_address(mb.output_address))
        dst[:] = src * 2 + layer
        mb.complete(0)
    mb.close()


def test_cpu_mailbox_between_processes():
    name = f"/xpool-test-mbox-{os.getpid()}"
    rows, hidden = 8, 16
    mb = rt.CpuMailbox.create(name, rows, hidden * 4)
    ctx = mp.get_context("fork")
    ready = ctx.Event()
    p = ctx.Process(target=_consumer, args=(name, rows, hidden * 4, 3, ready))
    p.start()
    try:
        assert ready.wait(10)
        assert mb.wait_status(rt.MBOX_IDLE, 5.0) == rt.WAIT_READY
        for layer in range(3):
            x = np.arange(5 * hidden, dtype=np.float32).reshape(5, hidden) + layer
            y = np.zeros_like(x)
            rc = mb.submit(x.ctypes.data, y.ctypes.data, 5, layer, rt.MODE_DECODE)
            assert rc == rt.RESULT_OK
            np.testing.assert_array_equal(y, x * 2 + layer)
        p.join(10)
        assert p.exitcode == 0
    finally:
        if p.is_alive():
            p.kill()
        mb.close()


def test_cpu_mailbox_consumer_that_never_answers_times_out_without_crashing():
    name = f"/xpool-test-mbox-to-{os.getpid()}"
    mb = rt.CpuMailbox.create(name, 4, 64)
    try:
        mb.activate()  # nobody will evaluate
        x = np.zeros((2, 16), dtype=np.float32)
        t0 = time.monotonic()
        rc = mb.submit(x.ctypes.data, x.ctypes.data, 2, 0, rt.MODE_DECODE, timeout_s=0.05)
        assert rc == rt.RESULT_TIMEOUT and time.monotonic() - t0 < 2
        assert mb.failure == rt.RESULT_TIMEOUT and mb.status == rt.MBOX_CLOSED
        # a closed mailbox refuses further submissions instead of hanging
        assert mb.submit(x.ctypes.data, x.ctypes.data, 2, 0, rt.MODE_DECODE, timeout_s=0.05) == rt.RESULT_PROTOCOL_MISMATCH
        assert mb.submit(x.ctypes.data, x.ctypes.data, 99, 0, rt.MODE_DECODE) == rt.RESULT_PROTOCOL_MISMATCH
    finally:
        mb.close()


def test_trace_buffer_drops_when_full_and_never_wraps():
    t = rt.TraceBuffer(4)
    for i in range(6):
        assert t.record(1, i, i * 2, 1000 + i) == (i < 4)
    n, dropped = t.counts()
    assert (n, dropped) == (4, 2)
    assert t.events() == [(1, i, i * 2, 1000 + i) for i in range(4)]


def test_dp_row_tables_follow_the_coordinators_admission_rules():
    """Scenarios of the reference's rendezvous inspection (src/cext/fabric/coordinator.cu:55-117) on the function
    that host and device share."""
    from crosspool_b200.native import runtime as rt

    P, D, I = rt.MODE_PREFILL, rt.MODE_DECODE, rt.MODE_IDLE
    # one rank: layout None, its rows are the payload, never idle
    assert rt.dp_inspect_rows(rt.DP_NONE, 7, [D], [7]) == (D, [0])
    assert rt.dp_inspect_rows(rt.DP_NONE, 7, [D], [6]) is None and rt.dp_inspect_rows(rt.DP_NONE, 7, [I], [7]) is None
    assert rt.dp_inspect_rows(rt.DP_UNIFORM_BY_RANK, 7, [D], [7]) is None        # a layout needs more than one rank
    assert rt.dp_inspect_rows(rt.DP_NONE, 8, [D, D], [4, 4]) is None             # ... and several ranks need a layout
    # uniform: equal (padded) counts, payload = ranks x count; an idle rank still holds its padded rows
    assert rt.dp_inspect_rows(rt.DP_UNIFORM_BY_RANK, 12, [D, P, I], [4, 4, 4]) == (P, [0, 4, 8])
    assert rt.dp_inspect_rows(rt.DP_UNIFORM_BY_RANK, 12, [D, D, D], [4, 4, 4]) == (D, [0, 4, 8])
    assert rt.dp_inspect_rows(rt.DP_UNIFORM_BY_RANK, 12, [D, D, D], [4, 5, 3]) is None
    assert rt.dp_inspect_rows(rt.DP_UNIFORM_BY_RANK, 13, [D, D, D], [4, 4, 4]) is None
    assert rt.dp_inspect_rows(rt.DP_UNIFORM_BY_RANK, 0, [D, D], [0, 0]) is None
    # packed: own counts back to back; idle exactly when a rank holds nothing; the counts sum to the payload
    assert rt.dp_inspect_rows(rt.DP_PACKED_BY_RANK, 9, [P, I, D], [6, 0, 3]) == (P, [0, 6, 6])
    assert rt.dp_inspect_rows(rt.DP_PACKED_BY_RANK, 9, [P, D, D], [6, 0, 3]) is None    # active rank without rows
    assert rt.dp_inspect_rows(rt.DP_PACKED_BY_RANK, 9, [P, I, D], [6, 1, 2]) is None    # idle rank with rows
    assert rt.dp_inspect_rows(rt.DP_PACKED_BY_RANK, 9, [P, D], [6, 4]) is None          # more rows than the payload
    assert rt.dp_inspect_rows(rt.DP_PACKED_BY_RANK, 9, [P, D], [6, 2]) is None          # fewer
    assert rt.dp_inspect_rows(rt.DP_PACKED_BY_RANK, 0, [I, I], [0, 0]) is None          # nobody has work
    assert rt.dp_inspect_rows(rt.DP_PACKED_BY_RANK, 4, [D, 3], [2, 2]) is None          # unknown forward mode


def test_records_are_checked_against_what_the_consumer_expects():
    from crosspool_b200.native import runtime as rt

    ok = dict(completed=4, capacity_rows=128, num_layers=28)
    assert rt.validate_invocation(16, 3, rt.MODE_DECODE, 5, **ok) == 0
    assert rt.validate_invocation(0, 3, rt.MODE_IDLE, 5, **ok) == 0                       # an idle step carries no rows
    for bad in (dict(rows=129), dict(rows=0), dict(layer=28), dict(mode=3), dict(sequence=6), dict(sequence=4)):
        a = dict(rows=16, layer=3, mode=rt.MODE_DECODE, sequence=5)
        a.update(bad)
        assert rt.validate_invocation(a["rows"], a["layer"], a["mode"], a["sequence"], **ok) == 2, bad
    assert rt.validate_invocation(16, 3, rt.MODE_DECODE, 5, requirement=7, **ok) == 2
    assert rt.validate_invocation(16, 3, rt.MODE_DECODE, 5, dp_layout=3, **ok) == 2
    assert rt.validate_completion(0, 16, 5, want_sequence=5, want_rows=16) == 0
    assert rt.validate_completion(0, 15, 5, want_sequence=5, want_rows=16) == 2           # rows differ
    assert rt.validate_completion(0, 16, 4, want_sequence=5, want_rows=16) == 2           # stale record
    assert rt.validate_completion(3, 0, 5, want_sequence=5, want_rows=16) == 3            # the producer's own failure code


def test_native_runtime_state_is_one_per_process():
    from crosspool_b200.native import runtime as rt

    rt.runtime_reset_for_tests()
    try:
        assert rt.runtime_state() == rt.NativeRuntimeState(False, None, None, {n: False for n in rt.DEBUG_OPTION_NAMES})
        rt.runtime_initialize("FfnAgent", 3, {"fabric_observer": True})
        st = rt.runtime_state()
        assert (st.initialized, st.role, st.device) == (True, "FfnAgent", 3)
        assert st.options == {"transport_observer": False, "fabric_observer": True, "graph_observer": False,
                              "ffn_routing_observer": False}
        rt.runtime_initialize("FfnAgent", 3, {"graph_observer": True})          # same identity: options replaced
        assert rt.runtime_state().options["graph_observer"] and not rt.runtime_state().options["fabric_observer"]
        with pytest.raises(RuntimeError, match="already initialised as FfnAgent on device 3"):
            rt.runtime_initialize("AtnAgent", 3)
        with pytest.raises(RuntimeError):
            rt.runtime_initialize("FfnAgent", 4)
        with pytest.raises(ValueError):
            rt.runtime_initialize("Scheduler", 0)
        rt.runtime_reset_for_tests()
        rt.runtime_initialize("Daemon", None)
        assert rt.runtime_state().device is None and rt.runtime_state().role == "Daemon"
    finally:
        rt.runtime_reset_for_tests()


def test_bootstrap_records_role_device_and_observer_switches_natively():
    from crosspool_b200 import bootstrap
    from crosspool_b200.config import load_config
    from crosspool_b200.native import runtime as rt

    bootstrap.reset_for_tests()
    try:
        cfg = load_config(env={"XPOOL_DEBUG_FABRIC_OBSERVER_ENABLE": "1"}, toml_text="[atn]\ndevices = [0]\n[ffn]\ndevices = [1]\n",
                          require=False)
        bootstrap.init("Instance", None, config=cfg)
        st = rt.runtime_state()
        assert st.role == "Instance" and st.device is None and st.options["fabric_observer"] and not st.options["graph_observer"]
        with pytest.raises(RuntimeError):
            bootstrap.init("FfnAgent", None, config=cfg)
    finally:
        bootstrap.reset_for_tests()
