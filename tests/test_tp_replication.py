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
