"""SGLang plugin: the same hosted-manifest contract over SGLang's memory pools (token-to-KV pool, per-request state
pools for recurrent layers). Reference counterpart: crates/kern-py/python/kern_sglang/model.py:1-312."""


def register() -> None:
    """The `sglang.srt.plugins` entry point: make `KernForCausalLM` known to SGLang's model registry."""
    from sglang.srt.models.registry import ModelRegistry

    from .model import KernForCausalLM

    ModelRegistry.models["KernForCausalLM"] = KernForCausalLM
