"""Small host-side utilities: model ids, process identity, CUDA error classes, device inventory,
background threads, signal handling, MPS endpoint description, bootstrap."""
import os
import signal
import subprocess
import sys
import threading
import time
import types

import pytest

from crosspool_b200 import bootstrap
from crosspool_b200.model import ModelId
from crosspool_b200.utils import background, cuda_errors, device, mps, procs, sighandler


def test_model_id_parses_and_round_trips_through_a_uri():
    m = ModelId.parse("Qwen/Qwen3-0.6B")
    assert (m.namespace, m.name) == ("Qwen", "Qwen3-0.6B") and str(m) == "Qwen/Qwen3-0.6B"
    assert m.uri() == "Qwen%2FQwen3-0.6B" and ModelId.from_uri(m.uri()) == m
    assert str(ModelId.parse("tiny")) == "tiny" and m.resolve("/models/") == "/models/Qwen/Qwen3-0.6B"
    for bad in ("", "a/b/c", "/x", "a b", "-x/y"):
        with pytest.raises(ValueError):
            ModelId.parse(bad)


def test_process_identity_tells_a_reused_pid_from_the_original_and_kills_exact_trees():
    me = procs.ProcUniqId.current()
    assert me.alive() and procs.ProcUniqId(me.pid, me.create_time - 100).status() == "replaced"
    child = subprocess.Popen([sys.executable, "-c", "import subprocess,sys,time; subprocess.Popen([sys.executable,'-c','import time; time.sleep(60)']); time.sleep(60)"])
    try:
        ident = procs.ProcUniqId.of(child.pid)
        for _ in range(100):
            if len(procs.tree(child.pid)) == 2:
                break
            time.sleep(0.05)
        pids = procs.kill_tree(ident, grace_s=3)
        assert len(pids) == 2 and pids[-1] == child.pid
        child.wait(5)
        assert procs.wait_exit(ident, 3) and ident.status() == "exited"
        assert procs.kill_tree(ident) == []     # an identity that is gone is never signalled again
    finally:
        if child.poll() is None:
            child.kill()


def test_cuda_error_classification():
    T = cuda_errors.is_terminal_device_error
    assert T(RuntimeError("CUDA error: an illegal memory access was encountered"))
    assert T(RuntimeError("CUDA error: unspecified launch failure"))
    assert not T(RuntimeError("CUDA out of memory. Tried to allocate 2 GiB"))
    assert not T(RuntimeError("CUDA error: operation not permitted when stream is capturing"))
    assert T(cuda_errors.CudaDriverError("cuLaunchKernel", 700)) and not T(cuda_errors.CudaDriverError("cuMemCreate", 2))
    assert not T(ValueError("bad shape"))


def test_device_inventory_and_visibility_mask():
    text = "0, GPU-aaaa, NVIDIA B200, 183359, 12\n1, GPU-bbbb, NVIDIA B200, 183359, 0\n"
    inv = device.parse_inventory(text)
    assert [d.uuid for d in inv] == ["GPU-aaaa", "GPU-bbbb"] and inv[0].memory_total_mib == 183359
    fake = lambda *a, **k: types.SimpleNamespace(returncode=0, stdout=text, stderr="")  # noqa: E731
    assert device.inventory(fake) == inv
    assert device.visible_indices(8, {"CUDA_VISIBLE_DEVICES": "3,1,9,2"}) == [3, 1]
    assert device.visible_indices(2, {}) == [0, 1]
    assert device.resolve_uuids([1], inv) == {1: "GPU-bbbb"}
    with pytest.raises(LookupError):
        device.resolve_uuids([5], inv)


def test_background_thread_runs_periodically_and_surfaces_errors():
    hits = []
    t = background.BackgroundThread.periodic(lambda: hits.append(1), 0.01, "tick").start()
    time.sleep(0.08)
    assert t.stop() and len(hits) >= 3
    t.check()

    def boom():
        raise KeyError("x")

    b = background.BackgroundThread.periodic(boom, 0.01, "boom").start()
    time.sleep(0.05)
    b.stop()
    with pytest.raises(RuntimeError, match="boom failed"):
        b.check()


def test_first_signal_requests_shutdown():
    got = []
    before = signal.getsignal(signal.SIGTERM)
    with sighandler.ShutdownSignals(on_request=got.append) as s:
        assert signal.getsignal(signal.SIGTERM) is not before          # the scope installs its own handler
        os.kill(os.getpid(), signal.SIGTERM)
        assert s.requested.wait(2) and got == [signal.SIGTERM] and s.signum == signal.SIGTERM
    assert signal.getsignal(signal.SIGTERM) == before                   # and puts the previous one back


def test_mps_endpoint_only_describes_an_environment():
    ep = mps.MpsEndpoint.for_device("GPU-12345678-abcd", root="/tmp/xp-mps-test")
    env = ep.client_env(active_thread_percentage=50)
    assert env["CUDA_MPS_PIPE_DIRECTORY"].endswith("/pipe") and env["CUDA_MPS_ACTIVE_THREAD_PERCENTAGE"] == "50"
    assert not ep.daemon_running()
    with pytest.raises(ValueError):
        ep.client_env(active_thread_percentage=0)
    e = {"CUDA_VISIBLE_DEVICES": "0"}
    with mps.MpsScope(ep, environ=e):
        assert e["CUDA_VISIBLE_DEVICES"] == "GPU-12345678-abcd"
    assert e == {"CUDA_VISIBLE_DEVICES": "0"}


def test_bootstrap_initialises_once_per_process():
    bootstrap.reset_for_tests()
    cfg = types.SimpleNamespace(logging_level="warning", logging_color="never", debug_transport_observer_enable=True)
    st = bootstrap.init("Instance", None, config=cfg)
    assert bootstrap.get_runtime_role() == "Instance" and [o.name for o in st.observers.observers] == ["transport"]
    assert bootstrap.init("Instance", None, config=cfg) is st
    with pytest.raises(RuntimeError):
        bootstrap.init("FfnAgent", 0, config=cfg)
    with pytest.raises(ValueError):
        bootstrap.reset_for_tests() or bootstrap.init("Nobody")
    bootstrap.reset_for_tests()


def test_owned_mps_scope_against_a_stand_in_control_binary(tmp_path):
    """The MPS control protocol without an MPS daemon: a stand-in for the control binary keeps server / client lists in
    memory and logs every invocation, so start-up, client termination with confirmation and shutdown are checked
    without touching how any GPU is shared."""
    import types

    log, state = [], {"servers": {4242: [111, 222]}, "sticky": set()}

    def fake_run(argv, input=None, env=None, **kw):
        assert env["CUDA_MPS_PIPE_DIRECTORY"].endswith("/pipe") and env["CUDA_VISIBLE_DEVICES"] == "GPU-abc"
        cmd = "-d" if "-d" in argv else (input or "").strip()
        log.append(cmd)
        out = ""
        if cmd == "get_server_list":
            out = "\n".join(str(s) for s in state["servers"])
        elif cmd.startswith("get_client_list"):
            out = "\n".join(str(c) for c in state["servers"].get(int(cmd.split()[1]), []))
        elif cmd.startswith("terminate_client"):
            _, s, c = cmd.split()
            if int(c) not in state["sticky"]:
                state["servers"][int(s)].remove(int(c))
        return types.SimpleNamespace(returncode=0, stdout=out, stderr="")

    ep = mps.MpsEndpoint.for_device("GPU-abc", root=tmp_path)
    scope = mps.OwnedMpsScope(ep, mps.MpsControl(ep, run=fake_run))
    scope.start()
    scope.start()                                   # idempotent
    assert log == ["-d"] and ep.pipe_dir.is_dir() and ep.log_dir.is_dir()
    assert scope.clients() == {4242: [111, 222]}
    assert scope.terminate_client(111) and scope.clients() == {4242: [222]}
    assert scope.terminate_client(999)              # not a client: nothing to do
    state["sticky"].add(222)
    assert not scope.terminate_client(222)          # still listed afterwards: not confirmed, the caller retains
    scope.stop()
    assert log[-1] == "quit" and not scope.started

    def failing(argv, **kw):
        return types.SimpleNamespace(returncode=1, stdout="", stderr="cannot create pipe")
    with pytest.raises(mps.MpsControlError, match="cannot create pipe"):
        mps.OwnedMpsScope(ep, mps.MpsControl(ep, run=failing)).start()


def test_atomic_write_replaces_whole_files_and_leaves_no_temporaries(tmp_path):
    from crosspool_b200.utils.files import atomic_write_text

    p = tmp_path / "sub" / "state.json"
    atomic_write_text(p, "one")
    atomic_write_text(p, "two")
    assert p.read_text() == "two"
    assert [f.name for f in p.parent.iterdir()] == ["state.json"]

    import os

    import pytest

    def refuse(*_a):
        raise OSError("no rename today")

    real, os.replace = os.replace, refuse          # the failure comes after the temporary file exists
    try:
        with pytest.raises(OSError):
            atomic_write_text(p, "three")
    finally:
        os.replace = real
    assert p.read_text() == "two"
    assert [f.name for f in p.parent.iterdir()] == ["state.json"]


def test_dtype_names_round_trip_and_reject_unknown_types():
    import pytest
    import torch

    from crosspool_b200.utils.dtype import decode_dtype, element_bytes, encode_dtype

    for name, dt in (("bfloat16", torch.bfloat16), ("float16", torch.float16), ("float32", torch.float32),
                     ("float8_e4m3fn", torch.float8_e4m3fn)):
        assert decode_dtype(name) is dt and encode_dtype(dt) == name and encode_dtype(name) == name
    assert decode_dtype("torch.bfloat16") is torch.bfloat16 and decode_dtype("BF16") is torch.bfloat16
    assert element_bytes("bf16") == 2 and element_bytes(torch.float8_e4m3fn) == 1
    with pytest.raises(ValueError):
        decode_dtype("float64x")
    with pytest.raises(ValueError):
        decode_dtype(torch.complex64)
    with pytest.raises(TypeError):
        decode_dtype(16)


def test_integers_are_range_checked_before_they_reach_native_code():
    import os

    import pytest

    from crosspool_b200.native import runtime as rt
    from crosspool_b200.utils.integer import ensure_sint64_nonnegative, ensure_uint32, ensure_uint64

    ensure_uint64(0, (1 << 64) - 1)
    ensure_uint32(0, (1 << 32) - 1)
    ensure_sint64_nonnegative(0, (1 << 63) - 1)
    for bad in (-1, 1 << 64):
        with pytest.raises(OverflowError):
            ensure_uint64(bad)
    with pytest.raises(OverflowError):
        ensure_sint64_nonnegative(1 << 63)
    with pytest.raises(OverflowError):
        ensure_uint32(1 << 32)
    for bad in (1.0, True, "3"):
        with pytest.raises(TypeError):
            ensure_uint64(bad)
    # the ECS channel refuses a negative quota instead of publishing 2**64 - 1 bytes
    ch = rt.EcsChannel.create(f"/xpool-int-{os.getpid()}", 1, 1)
    try:
        with pytest.raises(OverflowError):
            ch.publish_command(0, 1, -1)
        ch.publish_command(0, 1, 4096)
        assert ch.read_command(0) == (1, 4096)
    finally:
        ch.close()


def test_model_ids_follow_the_references_rules_for_canonical_components_and_order():
    """Vectors of the reference's identity test (tests/suites/unit/test_model.py): what is refused, how an id is
    written into a URI, and that ids sort as their text. A bare preset name without a namespace is this repository's
    own addition."""
    import pytest

    from crosspool_b200.model import ModelId

    m = ModelId.parse("Qwen/Qwen3-14B")
    assert (m.namespace, m.name, str(m), m.uri()) == ("Qwen", "Qwen3-14B", "Qwen/Qwen3-14B", "Qwen%2FQwen3-14B")
    assert m != "Qwen/Qwen3-14B" and len({m, ModelId.parse(str(m))}) == 1
    assert sorted((ModelId.parse("a/z"), ModelId.parse("a-/x"))) == [ModelId.parse("a-/x"), ModelId.parse("a/z")]
    for bad in ["/model", "org/", "org/a/b", "../model", "org/.", " org/model", "组织/model", ""]:
        with pytest.raises(ValueError):
            ModelId.parse(bad)
    with pytest.raises(Exception):
        m.name = "Other"            # frozen
