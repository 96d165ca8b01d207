"""Host-side logic of the GPU backends with the device calls replaced by fakes: what gets allocated, which handles are
published where. (The kernels and peer mappings themselves are covered by the GPU tests.)"""
import torch

from crosspool_b200 import config as C
from crosspool_b200.engine.atn_engine import EngineConfig
from crosspool_b200.parallel import fabric as F
from crosspool_b200.runtime import backends as B
from crosspool_b200.service.wire import FabricPlan

TOML = """
[atn]
devices = [0]
[ffn]
devices = [1, 2]
[scheduler.slo]
ttft_ms = 2000
tbt_ms = 50
[[models]]
id = "tiny-qwen3"
ffn_tp_size = 2
[[models]]
id = "tiny-qwen3-moe"
ffn_tp_size = 2
external = true
"""


class FakePeerBuffer:
    made: list = []

    def __init__(self, nbytes):
        self.nbytes, self.freed = nbytes, False
        FakePeerBuffer.made.append(self)

    def handle(self) -> bytes:
        return bytes([len(FakePeerBuffer.made)]) * 8

    def free(self):
        self.freed = True


def _plan(cfg) -> FabricPlan:
    from crosspool_b200.service.daemon.control import ControlPlane
    from crosspool_b200.service.wire import (AtnAgentRegistration, FfnAgentRegistration, InstanceFfnProfile, InstanceRankRegistration,
                                             ProcessRef)
    from crosspool_b200.native import EXPECTED_ABI

    cp = ControlPlane(cfg, process_alive=lambda ref: True)
    own = lambda pid: ProcessRef(abi_version=EXPECTED_ABI, pid=pid, create_time=1.0)
    cp.register_atnagent(AtnAgentRegistration(owner=own(10), device=0))
    for d in (1, 2):
        cp.register_ffnagent(FfnAgentRegistration(owner=own(20 + d), device=d, device_free_memory_bytes=64 << 30,
                                                  device_total_memory_bytes=180 << 30))
    for i, m in enumerate(("tiny-qwen3", "tiny-qwen3-moe")):
        cp.register_instance(InstanceRankRegistration(owner=own(10 if i == 0 else 99), model_id=m, rank=0, device=0,
                                                      ffn_profile=InstanceFfnProfile(max_prefill_rows=128, max_decode_rows=16, hidden_size=256)))
    return cp.fabric_plan()


def test_attention_backend_allocates_and_brokers_the_slot_of_an_external_rank_and_hosts_no_engine_for_it(monkeypatch):
    cfg = C.load_config(toml_text=TOML, env={})
    plan = _plan(cfg)
    assert sorted((r.model_id, r.rank) for r in plan.instance_ranks) == [("tiny-qwen3", 0), ("tiny-qwen3-moe", 0)]
    FakePeerBuffer.made = []
    monkeypatch.setattr(F, "PeerBuffer", FakePeerBuffer)
    monkeypatch.setattr(torch.cuda, "set_device", lambda *_: None)
    published = []
    backend = B.AtnBackend(cfg, 0, [("tiny-qwen3", 0)], EngineConfig(max_batch=16, prefill_chunk=128, max_seq_len=256), capacity_rows=128,
                           external=[("tiny-qwen3-moe", 0)], publish_arenas=lambda gen, arenas: published.append((gen, arenas)))
    handles = backend.prepare_join(plan)
    # one attention-side slot per rank, hosted or not, named in the plan for the FFN ranks to open
    assert set(handles) == {"atn:tiny-qwen3:0", "atn:tiny-qwen3-moe:0"} and len(FakePeerBuffer.made) == 2
    ext_place = B.placement_for(cfg, plan, "tiny-qwen3-moe", 0, backend.capacity_rows)
    assert FakePeerBuffer.made[1].nbytes == F.atn_slot_layout(ext_place).total_bytes > 0
    # ... and the external rank's slot handed to the daemon's broker, for the rank's own process to lease
    (gen, arenas), = published
    assert gen == plan.generation and [(a.model_id, a.rank, a.nbytes) for a in arenas] == [("tiny-qwen3-moe", 0, FakePeerBuffer.made[1].nbytes)]
    assert arenas[0].handle_hex == handles["atn:tiny-qwen3-moe:0"]
    assert set(backend.places) == {("tiny-qwen3", 0)}                 # no engine will be built for the external rank
    backend.finalize()
    assert all(b.freed for b in FakePeerBuffer.made)


def test_attention_backend_without_hosted_ranks_neither_warms_up_nor_listens(monkeypatch):
    cfg = C.load_config(toml_text=TOML.replace('id = "tiny-qwen3"\nffn_tp_size = 2\n', 'id = "tiny-qwen3"\nffn_tp_size = 2\nexternal = true\n'), env={})
    backend = B.AtnBackend(cfg, 0, [], EngineConfig(), external=[("tiny-qwen3", 0), ("tiny-qwen3-moe", 0)], listen=("127.0.0.1", 1))
    backend.warm_and_serve()
    assert backend.loop is None and backend.listener is None
    assert backend.poll_health() is None
