"""Hugging Face ``transformers`` models as the attention side of a disaggregated deployment.

``detach_ffn(model)`` does to a loaded ``*ForCausalLM`` what the serving-engine plugin does to the engine's model
classes (integrations/sglang/adapter.py; reference: src/xpool/integrations/sglang/models/qwen2.py:104-127): every
decoder layer's MLP (dense or MoE block; for OPT the ``fc1`` / activation / ``fc2`` triple) is replaced by a
parameter-free module that ships the post-attention-norm hidden states through ``torch.ops.xpool.ffn_shim`` and returns
what the FFN tier answers. The model keeps embeddings, attention, norms, residuals, KV cache and sampling; its own
``forward`` and ``generate`` run unchanged.

Where the operator leads depends on the tensor's device, exactly as for the plugin: on CUDA the native operator submits
to the Instance transport of the Fabric; on the CPU it calls the function installed with
``integrations.sglang.shim.bind_submit`` -- :func:`bind_cpu_tier` installs one that drives the mailboxes of a CPU FFN
tier (``engine/cpu_plumbing.py::FfnTierProcesses``).
"""

from .attach import DetachReport, HfFfnShim, bind_cpu_tier, detach_ffn, unbind

__all__ = ["DetachReport", "HfFfnShim", "bind_cpu_tier", "detach_ffn", "unbind"]
