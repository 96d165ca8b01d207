"""Public serving API: a set of co-located Instances stepped together.

``Deployment`` is what a user (and ``bench.py``) drives: add requests per model, call ``step()``,
read tokens. Each Instance is an :class:`AttentionEngine` whose FFN port decides where the FFN runs:

* :func:`build_loopback` — every role on one GPU, FFNs in-stream (1-GPU deployments);
* :func:`crosspool_b200.parallel.fabric.build_rank` — one process per GPU under ``torchrun``,
  attention ranks and FFN ranks connected by peer memory.

``step()`` launches one iteration of every Instance before collecting any of them, so Instances
overlap on the GPU(s): while one model's step waits for its FFN, another model's attention runs.
"""

from __future__ import annotations

import time
from dataclasses import dataclass, field

import torch

from .engine.atn_engine import AttentionEngine, EngineConfig, Sequence
from .engine.ffn_local import LocalFfnPort
from .models import config as model_config
from .models.config import ModelConfig
from .models.weights import random_attention_weights, random_ffn_weights


@dataclass
class InstanceHandle:
    model_id: str
    cfg: ModelConfig
    engine: AttentionEngine


@dataclass
class StepResult:
    tokens: dict[str, list[tuple[Sequence, int]]] = field(default_factory=dict)

    @property
    def num_tokens(self) -> int:
        return sum(len(v) for v in self.tokens.values())


class Deployment:
    def __init__(self, instances: list[InstanceHandle]):
        self.instances = instances
        self._by_id = {i.model_id: i for i in instances}

    def instance(self, model_id: str) -> InstanceHandle:
        return self._by_id[model_id]

    def warmup(self) -> None:
        for i in self.instances:
            i.engine.warmup()

    def add_request(self, model_id: str, prompt: list[int], max_new_tokens: int, arrival: float | None = None,
                    **sampling) -> Sequence:
        """``sampling``: ``temperature`` and ``seed`` (engines built with ``EngineConfig(sampling=True)``)."""
        return self._by_id[model_id].engine.add_request(prompt, max_new_tokens, arrival, **sampling)

    @property
    def has_work(self) -> bool:
        return any(i.engine.has_work for i in self.instances)

    def step(self) -> StepResult:
        """One iteration of every Instance that has work."""
        active = [i for i in self.instances if i.engine.has_work]
        self.idle_tick()
        for i in active:
            i.engine.launch_step()
        res = StepResult()
        for i in active:
            res.tokens[i.model_id] = i.engine.collect_step()
        return res

    def step_async(self, poll_s: float = 5e-5) -> StepResult:
        """Event-driven iteration for a serving loop: collects every Instance whose step has finished on the GPU and
        starts that Instance's next step at once; Instances whose step is still running are left alone. A 170 ms
        prefill chunk of a large model then no longer holds back the decode steps of the small model it shares the GPU
        with (``step`` runs the Instances in lockstep: every call lasts as long as the slowest of them). Returns the
        tokens of the steps collected in this call, possibly none."""
        res = StepResult()
        self.idle_tick()
        progressed = False
        waiting = []
        for i in self.instances:
            e = i.engine
            if e.step_in_flight:
                if not e.step_ready():
                    waiting.append(i)
                    continue
                progressed = progressed or getattr(e, "step_is_device_work", True)
                res.tokens[i.model_id] = e.collect_step()
            if e.has_work:
                e.launch_step()
                progressed = progressed or getattr(e, "step_is_device_work", True)
        if not progressed and not waiting:
            time.sleep(poll_s)          # every Instance with work is waiting for something on the host (KV capacity)
        elif not progressed and waiting:
            if len(waiting) == 1:       # nothing else to overlap with: wait for it (releases the interpreter lock)
                i = waiting[0]
                res.tokens[i.model_id] = i.engine.collect_step()
                if i.engine.has_work:
                    i.engine.launch_step()
            else:
                time.sleep(poll_s)
        return res

    def idle_tick(self) -> None:
        """Lets Instances without work serve their elastic-KV capacity commands."""
        for i in self.instances:
            tick = getattr(i.engine, "idle_tick", None)
            if tick is not None:
                tick()

    def run_until_idle(self, max_steps: int = 1 << 30) -> int:
        n = 0
        while self.has_work and n < max_steps:
            self.step()
            n += 1
        return n

    def stats(self) -> dict:
        out = {"h2d_bytes": 0, "d2h_bytes": 0, "launches": 0, "decode_steps": 0, "prefill_steps": 0}
        for i in self.instances:
            for k in out:
                out[k] += i.engine.stats[k]
        return out


def build_loopback(models: list[tuple[str, str | ModelConfig, int]], ecfg: EngineConfig | None = None,
                   device: str | torch.device = "cuda", tile_weights: bool = False) -> Deployment:
    """``models`` = [(instance id, preset name or ModelConfig, seed)]; random-init weights."""
    from .ops import gemm

    handles = []
    for model_id, preset, seed in models:
        cfg = preset if isinstance(preset, ModelConfig) else model_config.load(preset)
        aw = random_attention_weights(cfg, seed, device, torch.bfloat16)
        fw = random_ffn_weights(cfg, seed, device, torch.bfloat16)
        if tile_weights:
            for l in fw:
                if not l.is_moe:
                    l.gate_up, l.down = gemm.tile_weight(l.gate_up), gemm.tile_weight(l.down)
        eng = AttentionEngine(cfg, aw, LocalFfnPort(cfg, fw), ecfg, device)
        handles.append(InstanceHandle(model_id, cfg, eng))
    return Deployment(handles)


def percentile(values: list[float], p: float) -> float:
    """Linear-rank percentile ``(n - 1) * p / 100`` (the reference's definition,
    src/xpool-dev/xbench/harness/serving/measure.py:431-460)."""
    if not values:
        return float("nan")
    v = sorted(values)
    r = (len(v) - 1) * p / 100.0
    lo = int(r)
    hi = min(lo + 1, len(v) - 1)
    return v[lo] + (v[hi] - v[lo]) * (r - lo)


def now() -> float:
    return time.monotonic()
