"""Leader/follower request replication over a gloo group (two CPU processes, fake deployments)."""
import multiprocessing as mp
import os
import time
import types


class FakeDeployment:
    """Deterministic stand-in: every step emits (seq_id * 100 + step) for each running sequence."""

    def __init__(self):
        self.seqs, self.log, self._next = [], [], 0

    def add_request(self, model, prompt, max_new_tokens, **kw):
        if not prompt:
            raise ValueError("empty prompt")
        s = types.SimpleNamespace(seq_id=self._next, generated=[], max_new=max_new_tokens, finished=False)
        self._next += 1
        self.seqs.append(s)
        self.log.append(("add", model, tuple(prompt), max_new_tokens))
        return s

    @property
    def has_work(self):
        return any(not s.finished for s in self.seqs)

    def step(self):
        pairs = []
        for s in self.seqs:
            if not s.finished:
                s.generated.append(s.seq_id * 100 + len(s.generated))
                s.finished = len(s.generated) >= s.max_new
                pairs.append((s, s.generated[-1]))
        self.log.append(("step", len(pairs)))
        return types.SimpleNamespace(tokens={"m": pairs})


def _rank(rank, port, q):
    import torch.distributed as dist

    from crosspool_b200.runtime.tp_replication import TpEngineLoop

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=2)
    dep = FakeDeployment()
    loop = TpEngineLoop(dep, None, leader=rank == 0, idle_sleep=0.001)
    loop.start()
    out = None
    if rank == 0:
        time.sleep(0.05)
        a = loop.submit("m", [1, 2, 3], 3)
        bad = loop.submit("m", [], 2)
        b = loop.submit("m", [9], 2)
        got = []
        for p in (a, b):
            toks = []
            while True:
                item = p.out.get(timeout=10)
                toks.append(item[0])
                if item[1]:
                    break
            got.append(toks)
        err = bad.out.get(timeout=10)
        out = (got, type(err).__name__)
        loop.stop()
    else:
        loop._thread.join(20)
    q.put((rank, out, [e for e in dep.log if e[0] == "add"], loop.error))
    dist.destroy_process_group()


def test_followers_see_the_leaders_requests_in_order_and_stop_with_it():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + os.getpid() % 200
    ps = [ctx.Process(target=_rank, args=(r, port, q)) for r in (0, 1)]
    for p in ps:
        p.start()
    res = {}
    for _ in ps:
        r = q.get(timeout=60)
        res[r[0]] = r
    for p in ps:
        p.join(30)
    assert res[0][1] == ([[0, 1, 2], [100, 101]], "ValueError")
    assert res[0][2] == res[1][2] == [("add", "m", (1, 2, 3), 3), ("add", "m", (9,), 2)]
    assert res[0][3] is None and res[1][3] is None


class PerModelDeployment(FakeDeployment):
    """Tokens grouped by the model of each sequence, as a deployment with several Instances reports them."""

    def add_request(self, model, prompt, max_new_tokens, **kw):
        s = super().add_request(model, prompt, max_new_tokens, **kw)
        s.model = model
        return s

    def step(self):
        pairs = super().step().tokens["m"]
        out = {}
        for s, t in pairs:
            out.setdefault(s.model, []).append((s, t))
        return types.SimpleNamespace(tokens=out)


def _drain(p):
    toks = []
    while True:
        item = p.out.get(timeout=10)
        if isinstance(item, Exception):
            return item
        toks.append(item[0])
        if item[1]:
            return toks


def _mixed_rank(rank, port, q):
    import torch.distributed as dist

    from crosspool_b200.runtime.tp_replication import TpEngineLoop

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=2)
    dep = PerModelDeployment()
    loop = TpEngineLoop(dep, None, leader=rank == 0, idle_sleep=0.001, replicated={"m"})
    loop.start()
    time.sleep(0.05)
    if rank == 0:
        out = (_drain(loop.submit("m", [1, 2, 3], 3)), _drain(loop.submit("own0", [4], 2)))
        time.sleep(0.5)          # the follower's own request is served while the leader idles
        loop.stop()
    else:
        mine = _drain(loop.submit("own1", [7, 7], 4))
        refused = _drain(loop.submit("m", [5], 1))
        out = (mine, type(refused).__name__)
        loop._thread.join(20)
    q.put((rank, out, [e for e in dep.log if e[0] == "add"], loop.error))
    dist.destroy_process_group()


def test_a_rank_admits_requests_for_its_unreplicated_instances_itself_and_followers_refuse_replicated_ones():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29850 + os.getpid() % 100
    ps = [ctx.Process(target=_mixed_rank, args=(r, port, q)) for r in (0, 1)]
    for p in ps:
        p.start()
    res = {}
    for _ in ps:
        r = q.get(timeout=60)
        res[r[0]] = r
    for p in ps:
        p.join(30)
    assert res[0][3] is None and res[1][3] is None
    assert [len(t) for t in res[0][1]] == [3, 2]
    assert len(res[1][1][0]) == 4 and res[1][1][1] == "RuntimeError"
    # the replicated request reached both ranks; each rank's own request reached only that rank
    assert [e[1] for e in res[0][2]] == ["m", "own0"] and sorted(e[1] for e in res[1][2]) == ["m", "own1"]


def test_deployed_placement_names_the_tp_group_from_its_first_rank():
    """Every rank of an attention TP group resolves the same placement: the group's first rank talks to the FFN
    tier, the others follow it (reference: atn_tp_size in src/xpool/config.py)."""
    from crosspool_b200.config import load_config
    from crosspool_b200.runtime.backends import placement_for
    from crosspool_b200.service.wire import FabricPhase, FabricPlan, InstanceRankTopology, ShardPlacement

    cfg = load_config(env={}, toml_text="""
[daemon]
port = 18000
[atn]
devices = [0, 1]
[ffn]
devices = [2]
[scheduler.slo]
ttft_ms = 2000
tbt_ms = 50
[[models]]
id = "Qwen/Qwen3-0.6B"
atn_tp_size = 2
""")
    plan = FabricPlan(generation=1, uid="u", phase=FabricPhase.PREPARING_JOIN, atn_devices=[0, 1], ffn_devices=[2],
                      lanes_per_ffn_device=1, policy="fifo",
                      shards=[ShardPlacement(model_id="Qwen/Qwen3-0.6B", layer_begin=0, layer_end=28, tp_rank=0, tp_size=1,
                                             device=2, pe=2, bytes=1)],
                      instance_ranks=[InstanceRankTopology(model_id="Qwen/Qwen3-0.6B", rank=r, device=r, pe=r, instance_index=r)
                                      for r in (0, 1)])
    a, b = (placement_for(cfg, plan, "Qwen/Qwen3-0.6B", r, 256) for r in (0, 1))
    assert a == b and a.atn_rank == 0 and a.atn_tp_followers == (1,) and a.ffn_ranks == (2,)


def _agree_rank(rank, port, q):
    import torch.distributed as dist

    from crosspool_b200.ecs.reconciler import gloo_agreement

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=2)
    agree = gloo_agreement(None)
    out = [agree([rank, 10 + rank, 7]), agree([1, 3 - rank, 0])]
    q.put((rank, out))
    dist.destroy_process_group()


def test_gloo_agreement_gathers_every_ranks_vote():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29400 + os.getpid() % 200
    ps = [ctx.Process(target=_agree_rank, args=(r, port, q)) for r in (0, 1)]
    for p in ps:
        p.start()
    res = dict(q.get(timeout=60) for _ in ps)
    for p in ps:
        p.join(30)
    assert res[0] == res[1] == [[[0, 10, 7], [1, 11, 7]], [[1, 3, 0], [1, 2, 0]]]
