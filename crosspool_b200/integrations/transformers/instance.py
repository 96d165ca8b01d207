"""A ``transformers`` model as an Instance rank in a process of its own, inside a deployment run by the daemon.

This is the reference's process model (an engine process per Instance rank, an attention agent that brokers its
Transport arena, FFN agents, one daemon; src/xpool/runtime/instance.py, src/xpool/integrations/sglang/hooks/lifecycle.py)
with the library model standing where the serving engine stands:

    register -> wait until the generation is executable -> lease the arena from the daemon -> map the FFN ranks' arenas
    -> detach the decoder FFNs and bind ``torch.ops.xpool.ffn_shim`` -> publish *initialised* -> wait for system ready

after which the model's own ``forward`` / ``generate`` run attention here and every FFN on the tier. ``leave()`` retires
the rank in order. The data plane is the CPU one (a deployment started with ``--backend cpu`` and the model marked
``external = true``); on GPUs the same sequence ends in ``integrations.sglang.transport.FabricInstanceTransport``.
"""

from __future__ import annotations

from ...config import XpoolConfig
from ...runtime.instance import InstanceRankRuntime
from ...service.client import XpoolClient, self_ref
from ...service.wire import InstanceFfnProfile
from .attach import DetachReport, bind_cpu_tier, detach_ffn, unbind


class ExternalInstance:
    def __init__(self, cfg: XpoolConfig, model_id: str, rank: int = 0, client: XpoolClient | None = None):
        from ...native import EXPECTED_ABI
        from ...runtime.cpu_backends import cpu_capacity_rows

        self.cfg, self.model_id, self.rank, self.capacity_rows = cfg, model_id, rank, cpu_capacity_rows(cfg)
        if not cfg.model(model_id).external:
            raise ValueError(f"model {model_id!r} is not marked external in the deployment's configuration")
        self.client = client or XpoolClient(cfg.daemon_host, cfg.daemon_port)
        self.owner = self_ref(EXPECTED_ABI)
        self.device = cfg.atn_devices[rank]
        self.runtime: InstanceRankRuntime | None = None
        self.report: DetachReport | None = None

    def join(self, model, timeout_s: float = 120.0, listener: tuple[str, int] | None = None) -> DetachReport:
        """Runs the start-up sequence for ``model`` (a loaded ``*ForCausalLM``) and returns what was detached.
        ``listener``: the (host, port) this rank serves requests on, published with *initialised*."""
        from ...runtime.cpu_backends import attach_cpu_instance

        self.client.check_config(self.owner, self.cfg.digest())
        shape = self.cfg.model_shape(self.model_id)
        rows = self.cfg.engine_max_rows if next(model.parameters()).is_cuda else self.capacity_rows
        profile = InstanceFfnProfile(max_prefill_rows=rows, max_decode_rows=rows, hidden_size=shape.hidden_size)
        on_gpu = next(model.parameters()).is_cuda

        def attach_gpu(binding, plan):
            # The GPU form of the same step: map the leased attention-side slot and the FFN ranks' slots by their IPC
            # handles and point the native operator at them. Written against the brokering of AtnBackend; it has not
            # run on GPUs yet (the CPU form below is what the tests exercise).
            from ...runtime.backends import placement_for
            from ..sglang.transport import FabricInstanceTransport

            place = placement_for(self.cfg, plan, self.model_id, self.rank, self.cfg.engine_max_rows)
            t = FabricInstanceTransport.from_handles(place, binding.handle_hex,
                                                     [plan.slot_handles[f"ffn:{self.model_id}:{self.rank}:{pe}"] for pe in place.ffn_ranks],
                                                     next(model.parameters()).device)
            t.make_current()
            return t

        rt = InstanceRankRuntime(self.client, self.model_id, self.rank, self.device, profile, owner=self.owner,
                                 attach=attach_gpu if on_gpu else
                                 (lambda binding, plan: attach_cpu_instance(self.cfg, plan, self.model_id, self.rank)))
        self.runtime = rt
        rt.start()
        plan = rt.wait_for_fabric_executable(timeout_s=timeout_s)
        transport = rt.attach_arena_from_daemon(plan)
        self.report = detach_ffn(model)
        if not on_gpu:
            bind_cpu_tier(transport.port)
        rt.publish_initialized(listener)
        rt.wait_for_ready(timeout_s=timeout_s)
        return self.report

    @property
    def ffn_calls(self) -> int:
        port = getattr(getattr(self.runtime, "transport", None), "port", None)
        return port.calls if port is not None else 0

    def leave(self) -> bool:
        unbind()
        return self.runtime.detach() if self.runtime is not None else True
