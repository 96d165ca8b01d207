"""Sealed creation and ordered retirement of a serving engine's child processes, with real (sleeping) children."""
import signal
import subprocess
import sys
import time

import pytest

from crosspool_b200.integrations.sglang.shutdown import OwnerRetained, ProcessTreeRetirement
from crosspool_b200.utils.procs import ProcUniqId


def _child(ignore_term: bool = False):
    code = "import signal,time\n" + ("signal.signal(signal.SIGTERM, signal.SIG_IGN)\n" if ignore_term else "") + "time.sleep(120)\n"
    return subprocess.Popen([sys.executable, "-c", code])


def _reap(*procs):
    for p in procs:
        try:
            p.kill()
        except Exception:
            pass
        p.wait(10)


def test_importers_are_forced_before_exporters_are_asked_to_leave():
    order = []
    imp = [_child(), _child()]
    exp = [_child()]
    try:
        asked = []
        r = ProcessTreeRetirement(request_shutdown=asked.append, cleanup_timeout_s=6.0, termination_timeout_s=5.5,
                                  confirm_context=lambda targets, deadline: order.append([t.pid for t in targets]))
        r.launch(lambda: (r.creating(lambda: imp), r.creating(lambda: exp[0], exporters=True)))
        assert [p.pid for p in r.importers] == [p.pid for p in imp] and [p.pid for p in r.exporters] == [exp[0].pid]
        t0 = time.monotonic()
        r.retire()
        assert time.monotonic() - t0 < 6.0 and len(asked) == 1 and not r.retained
        assert all(p.wait(5) == -signal.SIGKILL for p in imp)          # importers did not leave by themselves: forced
        assert exp[0].wait(5) == -signal.SIGTERM                        # the exporter was asked, after its consumers left
        assert order == [[p.pid for p in imp] + [exp[0].pid]]           # context confirmation saw importers first
        r.retire()                                                      # idempotent once everything is gone
        assert len(asked) == 1
    finally:
        _reap(*imp, *exp)


def test_a_failed_generation_skips_the_cooperative_wait_and_an_exporter_that_ignores_term_is_killed():
    imp, exp = _child(), _child(ignore_term=True)
    try:
        time.sleep(0.3)      # let the exporter install its handler
        r = ProcessTreeRetirement(cleanup_timeout_s=30.0, termination_timeout_s=1.0)
        r.creating(lambda: imp)
        r.creating(lambda: exp, exporters=True)
        r.failed = True
        t0 = time.monotonic()
        r.retire(wait_timeout_s=1.0)
        assert time.monotonic() - t0 < 6.0           # no 29 s of cooperative waiting
        assert imp.wait(5) == -signal.SIGKILL and exp.wait(5) == -signal.SIGKILL
    finally:
        _reap(imp, exp)


def test_unsealed_creation_retains_the_owner_and_touches_nothing():
    survivor = _child()
    try:
        r = ProcessTreeRetirement(cleanup_timeout_s=2.0, termination_timeout_s=1.0)
        r.creating(lambda: survivor)

        def broken_factory():
            raise OSError("spawn failed half way")

        with pytest.raises(OSError):
            r.creating(broken_factory)
        assert r.creation_unconfirmed
        with pytest.raises(OwnerRetained, match="never sealed"):
            r.retire()
        assert r.retained and survivor.poll() is None         # nothing was signalled
        assert r.as_step()(1.0) is False
    finally:
        _reap(survivor)


def test_a_signal_during_creation_is_raised_only_after_the_factory_has_unwound():
    made = []
    r = ProcessTreeRetirement(cleanup_timeout_s=3.0, termination_timeout_s=2.5)

    def factory():
        p = _child()
        made.append(p)
        r.note_signal(signal.SIGTERM)          # the signal handler runs while the factory is busy
        return p

    try:
        with pytest.raises(SystemExit) as e:
            r.launch(lambda: r.creating(factory))
        assert e.value.code == 128 + signal.SIGTERM
        assert r.importers and r.importers[0].pid == made[0].pid    # the handle was recorded before the exit
        assert made[0].wait(5) == -signal.SIGKILL                   # ... and the launch failure retired it
        with pytest.raises(SystemExit):
            r.creating(lambda: _child())                            # nothing new is created after a cancellation
    finally:
        _reap(*made)


def test_identity_includes_the_creation_time_so_a_recycled_pid_is_never_signalled():
    p = _child()
    try:
        ident = ProcUniqId(p.pid, ProcUniqId.of(p.pid).create_time - 100.0)    # "an earlier process with this pid"
        assert ident.status() == "replaced"
        r = ProcessTreeRetirement(cleanup_timeout_s=1.0, termination_timeout_s=0.5)
        r.importers.append(ident)
        r.retire()
        assert p.poll() is None
    finally:
        _reap(p)


def test_hooks_name_the_engine_seams_and_wrap_the_factories():
    r = ProcessTreeRetirement()
    hooks = {h.target.rsplit(".", 1)[-1]: h for h in r.hooks()}
    assert set(hooks) == {"_launch_subprocesses", "_launch_scheduler_processes", "spawn_weight_cache_daemon", "kill_process_tree"}
    p = _child()
    try:
        out = hooks["_launch_scheduler_processes"].handler(lambda tag: [p], "x")
        assert out == [p] and r.importers[0].pid == p.pid
    finally:
        _reap(p)
