"""The attention backend vLLM is told to use: it allocates the paged KV in the layout the manifest's attention kernels
read ([pages, 2, kv_heads, block, head_dim], block 64) and does no attention math of its own — the manifest's
programs append to and read the cache themselves.
Reference counterpart: crates/kern-py/python/kern_vllm/backend.py:27-109 (KERNEL_BLOCK = 64, no-op backends)."""
from __future__ import annotations

KERNEL_BLOCK = 64


class KernAttentionBackend:
    accept_output_buffer = True

    @staticmethod
    def get_name() -> str:
        return "KERN_B200"

    @staticmethod
    def get_supported_kernel_block_size() -> list[int]:
        return [KERNEL_BLOCK]

    @staticmethod
    def get_kv_cache_shape(num_blocks: int, block_size: int, num_kv_heads: int, head_size: int, cache_dtype_str: str = "auto"):
        if block_size != KERNEL_BLOCK:
            raise ValueError(f"the attention kernels read {KERNEL_BLOCK}-token pages, not {block_size}")
        return (num_blocks, 2, num_kv_heads, block_size, head_size)

    @staticmethod
    def get_impl_cls():
        return KernAttentionImpl

    @staticmethod
    def get_builder_cls():
        return KernMetadataBuilder


class KernAttentionImpl:
    """Never computes: the layer's attention ran inside the manifest's program."""

    def __init__(self, *a, **kw):
        pass

    def forward(self, layer, query, key, value, kv_cache, attn_metadata, output=None, **kw):
        return output if output is not None else query


class KernMetadataBuilder:
    """Passes vLLM's common metadata through: positions, slot mapping, block table, sequence lengths and the
    query-start offsets are all the manifest's inputs need."""

    def __init__(self, *a, **kw):
        pass

    def build(self, common_prefix_len, common_attn_metadata, fast_build: bool = False):
        return common_attn_metadata
