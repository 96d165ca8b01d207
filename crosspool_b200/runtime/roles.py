"""The two agent roles.

``FfnAgent`` owns one FFN device: it registers its free memory and GEMM device properties, loads the
shards the plan assigns to it, publishes its slot arenas, installs and starts the Executor Lanes.
``AtnAgent`` owns one attention device and *hosts the Instances placed on it* (engine, KV cache,
request API): in the reference the Instances are separate SGLang processes that reach the AtnAgent
through a same-GPU mailbox under MPS (src/xpool/runtime/atnagent.py, instance.py); here a mailbox
between two processes on one GPU would mean kernels of different launches waiting on one another on
the same device, which this system never does, so the attention role is one process per GPU.
"""

from __future__ import annotations

from ..service.wire import (AtnAgentRegistration, FabricPlan, FfnAgentRegistration, GemmDeviceProperties,
                            InstanceFfnProfile, InstanceRankInitialized, InstanceRankRegistration)
from .agent import Agent


class FfnAgent(Agent):
    role = "ffnagent"

    def __init__(self, client, device, backend, free_bytes: int, total_bytes: int, model_specs=None,
                 props: GemmDeviceProperties | None = None, **kw):
        super().__init__(client, device, backend, **kw)
        self.free_bytes, self.total_bytes = free_bytes, total_bytes
        self.model_specs = model_specs or []
        self.props = props or GemmDeviceProperties()

    def register(self) -> None:
        self.client.register_ffnagent(FfnAgentRegistration(
            owner=self.owner, device=self.device, device_free_memory_bytes=self.free_bytes,
            device_total_memory_bytes=self.total_bytes, model_specs=self.model_specs, device_properties=self.props))

    def heartbeat(self):
        return self.client.heartbeat_ffnagent(self.device, self.owner)

    def find_pe(self, plan: FabricPlan) -> int:
        return len(plan.atn_devices) + plan.ffn_devices.index(self.device)


class AtnAgent(Agent):
    role = "atnagent"

    def __init__(self, client, device, backend, instances: list[tuple[str, int, InstanceFfnProfile]], **kw):
        """``instances``: (model id, rank, FFN profile) of the Instance ranks this device hosts."""
        super().__init__(client, device, backend, **kw)
        self.instances = instances
        self._initialized = False

    def register(self) -> None:
        self.client.register_atnagent(AtnAgentRegistration(owner=self.owner, device=self.device))
        for model_id, rank, prof in self.instances:
            self.client.register_instance(InstanceRankRegistration(owner=self.owner, model_id=model_id, rank=rank,
                                                                   device=self.device, ffn_profile=prof))

    def heartbeat(self):
        for model_id, rank, _ in self.instances:
            self.client.heartbeat_instance(model_id, rank, self.owner)
        return self.client.heartbeat_atnagent(self.device, self.owner)

    def find_pe(self, plan: FabricPlan) -> int:
        return plan.atn_devices.index(self.device)

    def advance(self):
        fp = super().advance()
        from ..service.wire import FabricPhase

        if fp == FabricPhase.EXECUTABLE and not self._initialized and not self.failed:
            warm = getattr(self.backend, "warm_and_serve", None)
            if warm is not None:
                warm()  # engine graphs invoke the FFN tier, so they are captured only now
            listener = getattr(self.backend, "listener", None)
            for model_id, rank, _ in self.instances:
                self.client.instance_initialized(model_id, InstanceRankInitialized(
                    owner=self.owner, rank=rank, generation=self.generation, serving_listener=listener))
            self._initialized = True
        return fp
