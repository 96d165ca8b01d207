"""Request replication for an Instance whose attention runs tensor-parallel over several processes.

Every attention TP rank runs the same engine on its share of the heads and must see the same requests
in the same order at the same step, or the ranks' schedules (and their peer-memory handshakes) diverge.
The leader (TP rank 0) owns the HTTP front end; once per engine step it broadcasts the requests that
arrived since the last step over a ``torch.distributed`` CPU group; followers add them to their own
deployment before stepping. The broadcast also carries the stop signal, so all ranks leave together.
(The reference relies on its serving engine's scheduler broadcast for the same purpose.)

A device may also host Instances that are not tensor-parallel (a data-parallel rank of another model). When the loop
is told which models are replicated, requests for the others are admitted by the rank that received them, on any rank,
and never broadcast: the ranks' loops then differ in what else they step, but still exchange once per iteration and
step the replicated Instances in the same iterations.
"""

from __future__ import annotations


from .serving import EngineLoop, Pending


class TpEngineLoop(EngineLoop):
    def __init__(self, deployment, group, leader: bool, idle_sleep: float = 0.0005, replicated: set[str] | None = None):
        super().__init__(deployment, idle_sleep)
        self.group, self.leader = group, leader
        self.replicated = replicated        # None: every request is replicated (every hosted Instance is tensor-parallel)

    def _exchange(self, batch: list[dict] | None, stop: bool) -> tuple[list[dict], bool]:
        import torch.distributed as dist

        box = [{"requests": batch or [], "stop": stop}] if self.leader else [None]
        dist.broadcast_object_list(box, src=dist.get_global_rank(self.group, 0) if self.group is not None else 0, group=self.group)
        return box[0]["requests"], box[0]["stop"]

    def _run(self) -> None:
        hosted = {i.model_id for i in getattr(self.dep, "instances", ())} or None
        try:
            while True:
                mine: list[Pending] = []
                local: list[Pending] = []
                if self.leader or self.replicated is not None:
                    while not self._inbox.empty():
                        p = self._inbox.get_nowait()
                        if self.replicated is not None and p.model_id not in self.replicated:
                            local.append(p)
                        elif self.leader:
                            mine.append(p)
                        else:
                            p.deliver(RuntimeError(f"{p.model_id} is served by its tensor-parallel leader, not by this rank"))
                reqs, stop = self._exchange(
                    [{"model": p.model_id, "prompt": p.prompt, "max_new_tokens": p.max_new_tokens, "temperature": p.temperature,
                      "seed": p.seed} for p in mine] if self.leader else None, self._stop.is_set())
                if stop:
                    for p in local:
                        p.deliver(RuntimeError("the engine loop is stopping"))
                    break
                for i, r in enumerate(reqs):
                    if hosted is not None and r["model"] not in hosted:
                        continue       # an Instance that only the leader's device hosts
                    kw = {"temperature": r["temperature"], "seed": r["seed"]} if r["temperature"] > 0 else {}
                    try:
                        seq = self.dep.add_request(r["model"], r["prompt"], r["max_new_tokens"], **kw)
                        if self.leader:
                            self._by_seq[(r["model"], seq.seq_id)] = mine[i]
                    except Exception as e:   # every rank refuses the same request the same way
                        if self.leader:
                            mine[i].deliver(e)
                for p in local:
                    kw = {"temperature": p.temperature, "seed": p.seed} if p.temperature > 0 else {}
                    try:
                        seq = self.dep.add_request(p.model_id, p.prompt, p.max_new_tokens, **kw)
                        self._by_seq[(p.model_id, seq.seq_id)] = p
                    except Exception as e:
                        p.deliver(e)
                if not self.dep.has_work:
                    self._idle()       # the same number of idle ticks on every rank: one per exchange
                    continue
                res = self.dep.step()
                self.steps += 1
                if not self.leader and self.replicated is None:
                    continue
                for model_id, pairs in res.tokens.items():
                    for seq, tok in pairs:
                        p = self._by_seq.get((model_id, seq.seq_id))
                        if p is None:
                            continue
                        done = seq.finished
                        p.deliver((tok, done))
                        self.tokens += 1
                        if done:
                            del self._by_seq[(model_id, seq.seq_id)]
        except Exception as e:
            self.error = e
            for p in self._by_seq.values():
                p.deliver(e)
