"""Daemon-side ECS service: channel per generation, freeze once every rank and device has reported,
then policy ticks that move capacity; over the real seqlock channel with fake-driver reconcilers."""
import types

from crosspool_b200.ecs import reconciler as R
from crosspool_b200.ecs import vmm
from crosspool_b200.models import config as mc
from crosspool_b200.native.runtime import EcsChannel
from crosspool_b200.service.daemon.ecs_service import EcsService
from crosspool_b200.service.wire import FabricPhase


def _plan(gen=1):
    ranks = [types.SimpleNamespace(model_id=m, rank=0, device=0) for m in ("a/x", "b/y")]
    return types.SimpleNamespace(generation=gen, atn_devices=[0], instance_ranks=ranks)


def test_service_opens_freezes_and_arbitrates():
    cp = types.SimpleNamespace(generation=None)
    published = []
    svc = EcsService(cp, published.append, utilization=1.0)
    assert svc.tick() is None and svc.channel is None                 # no generation yet
    cp.generation = types.SimpleNamespace(number=1, phase=FabricPhase.PREPARING_EXECUTION, plan=_plan())
    svc.tick()
    ref = published[-1]
    assert ref.generation == 1 and ref.partitions == {"a/x:0": 0, "b/y:0": 1} and ref.devices == {"0": 0}
    # agent side: attach, describe partitions, report the device
    ch = EcsChannel.attach(ref.name)
    cfg = mc.preset("Qwen/Qwen3-0.6B")
    ppb, _ = vmm.bundle_geometry(cfg, 16)
    q, drv = vmm.MemoryQuota(1 << 50), vmm.Driver.fake(1 << 50)
    recs = []
    for idx in (0, 1):
        kv = vmm.elastic_kv_cache(cfg, 4 * ppb, 16, "cpu", drv, q, initial_bundles=1, make_tensors=False)
        bb = kv.backing.bundle_bytes
        ch.set_partition(idx, 0, 0, 0, bb, kv.backing.bundle_count * bb)
        recs.append(R.CapacityReconciler(kv, ch, idx))
        svc.tick()
        assert not svc.frozen                                          # device report still missing
    ch.publish_report(0, 2 * bb, 100 * bb, 1)                          # two spare bundles besides the two floors
    svc.tick()
    assert svc.frozen
    for r in recs:
        r.poll()
    assert [r.mapped_bundles for r in recs] == [2, 2]
    # rank 0 needs two more bundles; rank 1 is idle and gives one back
    recs[0].publish_demand(2 * ppb)
    for _ in range(10):
        svc.tick()
        for r in recs:
            r.poll()
    assert [r.mapped_bundles for r in recs] == [3, 1]
    # the generation stops: the channel goes away and the reference is withdrawn
    cp.generation.phase = FabricPhase.STOPPED
    svc.tick()
    assert svc.channel is None and published[-1] is None
    ch.close()
