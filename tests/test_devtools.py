"""Supervisor (owned process groups, retirement, leases, ports) and the xtest runner over the case catalogue."""
import subprocess
import sys
import types

import pytest

from crosspool_b200.devtools import xtest
from crosspool_b200.devtools.supervisor import DeviceLeases, Supervisor, reserve_port


def test_supervisor_retires_in_reverse_order_and_kills_what_ignores_sigterm(tmp_path):
    with Supervisor(tmp_path) as sup:
        a = sup.start("sleeper", [sys.executable, "-c", "import time; time.sleep(60)"], retire_deadline_s=5)
        b = sup.start("stubborn", [sys.executable, "-c", "import signal,time; signal.signal(signal.SIGTERM, signal.SIG_IGN); print('up', flush=True); time.sleep(60)"],
                      retire_deadline_s=0.5)
        sup.wait_until(lambda: b.log.read_text().strip() == "up", 10, what="stubborn child up")
        assert sup.poll() == {"sleeper": None, "stubborn": None}
        codes = sup.retire_all()
    assert codes["sleeper"] == -15 and codes["stubborn"] == -9
    assert [e for e in sup.events if e[0] != "start"] == [("kill", "stubborn"), ("retired", "stubborn"), ("retired", "sleeper")]
    assert a.proc.poll() is not None


def test_wait_until_fails_early_when_a_child_dies(tmp_path):
    with Supervisor() as sup:
        sup.start("bad", [sys.executable, "-c", "raise SystemExit(3)"])
        with pytest.raises(RuntimeError, match="bad exited with code 3"):
            sup.wait_until(lambda: False, 10, what="never")


def test_device_leases_are_exclusive_and_ports_are_free():
    leases = DeviceLeases([0, 1, 2])
    with leases.lease("case-a", 2) as a:
        assert a == [0, 1] and leases.acquire("case-b", 2) is None
        with leases.lease("case-c", 1) as c:
            assert c == [2]
    assert leases.free == [0, 1, 2]
    p = reserve_port()
    assert 1024 < p < 65536


def test_xtest_catalogue_and_runner_lease_devices_and_skip_what_does_not_fit():
    cases = xtest.load_cases()
    names = [c.name for c in cases]
    assert names[0] == "unit-host" and {"kernels", "topology-atn1-ffn2", "deployed-stack"} <= set(names)
    topo = next(c for c in cases if c.name == "topology-atn1-ffn2")
    assert topo.gpus == 3 and topo.tier == "multigpu" and dict(topo.env)["NCCL_NVLS_ENABLE"] == "0"
    seen = {}

    def fake_run(cmd, env=None, **kw):
        seen["cmd"], seen["devices"] = cmd, env.get("CUDA_VISIBLE_DEVICES")
        return types.SimpleNamespace(returncode=0, stdout="3 passed in 1.0s\n", stderr="")

    res = xtest.run_case(topo, DeviceLeases([4, 5, 6, 7]), runner=fake_run)
    assert res["status"] == "passed" and seen["devices"] == "4,5,6" and seen["cmd"][-2:] == ["-m", "gpu"] and res["summary"] == "3 passed in 1.0s"
    assert xtest.run_case(topo, DeviceLeases([0]), runner=fake_run)["status"] == "skipped"

    def failing(cmd, **kw):
        raise subprocess.TimeoutExpired(cmd, 1)
    assert xtest.run_case(cases[0], DeviceLeases([]), runner=failing)["rc"] == 124


def test_supervised_task_reports_how_it_ended_and_retires_a_grandchild_that_left_its_group(tmp_path):
    """The task starts a grandchild in a session of its own and exits: killing the task's group cannot reach it, but
    the supervising process adopted it (child subreaper) and drains it by identity."""
    import subprocess
    import sys
    import textwrap

    import psutil

    code = textwrap.dedent("""
        import subprocess, sys, time
        g = subprocess.Popen([sys.executable, "-c", "import time; time.sleep(120)"], start_new_session=True)
        print("grandchild", g.pid, flush=True)
        time.sleep(0.3)
    """)
    runner = textwrap.dedent(f"""
        import json, sys
        from crosspool_b200.devtools.supervisor import Supervisor
        sup = Supervisor(log_dir={str(tmp_path)!r}, adopt_orphans=True)
        c = sup.run("task", [sys.executable, "-c", {code!r}], timeout_s=20)
        slow = sup.run("slow", [sys.executable, "-c", "import time; time.sleep(60)"], timeout_s=0.5)
        bad = sup.run("bad", [sys.executable, "-c", "raise SystemExit(7)"], timeout_s=20)
        print(json.dumps(dict(kind=c.kind, rc=c.exit_code, orphans=list(c.orphans), ok=c.ok, tail=c.log_tail,
                              slow=slow.kind, bad=[bad.kind, bad.exit_code])))
    """)
    # in a process of its own: becoming a subreaper is for the life of the process
    r = subprocess.run([sys.executable, "-c", runner], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stderr[-2000:]
    import json

    out = json.loads(r.stdout.strip().splitlines()[-1])
    assert out["kind"] == "completed" and out["rc"] == 0 and not out["ok"]        # it finished, but left a process behind
    gpid = int(out["tail"].split()[1])
    assert out["orphans"] == [gpid]
    try:
        assert psutil.Process(gpid).status() == psutil.STATUS_ZOMBIE      # at most an unreaped entry, never a live process
    except psutil.NoSuchProcess:
        pass
    assert out["slow"] == "timed_out" and out["bad"] == ["failed", 7]


def test_xtest_case_under_the_supervisor_times_out_as_a_group(tmp_path):
    from crosspool_b200.devtools import xtest
    from crosspool_b200.devtools.supervisor import DeviceLeases, Supervisor

    (tmp_path / "test_sleepy.py").write_text("import time\ndef test_sleep():\n    time.sleep(60)\n")
    (tmp_path / "test_quick.py").write_text("def test_ok():\n    assert True\n")
    sup = Supervisor(log_dir=tmp_path / "logs")
    slow = xtest.run_case(xtest.TestCase("sleepy", "cpu", (str(tmp_path / "test_sleepy.py"),), timeout_s=3.0), DeviceLeases([]),
                          supervisor=sup)
    assert slow["status"] == "failed" and slow["ended"] == "timed_out" and "timed out after 3 s" in slow["summary"]
    quick = xtest.run_case(xtest.TestCase("quick", "cpu", (str(tmp_path / "test_quick.py"),), timeout_s=120.0), DeviceLeases([]),
                           supervisor=sup)
    assert quick["status"] == "passed" and quick["ended"] == "completed" and "1 passed" in quick["summary"]
