"""vLLM plugin: serves a kern_b200 manifest as a vLLM model. vLLM keeps its scheduler, KV-cache manager and
sampler; the forward pass (every layer, attention included) is the manifest's programs on hand-written sm_100a
kernels, enqueued on vLLM's stream. Register with ``vllm.ModelRegistry`` through the ``vllm.general_plugins`` entry
point (``kern_vllm:register``). Reference counterpart: crates/kern-py/python/kern_vllm/{model,backend}.py."""


def register() -> None:
    from vllm import ModelRegistry

    ModelRegistry.register_model("KernForCausalLM", "kern_vllm.model:KernForCausalLM")
