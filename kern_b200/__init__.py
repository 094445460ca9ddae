"""kern_b200: a Blackwell-native (sm_100a), manifest-driven LLM inference engine.

A model ships as a package: ``manifest.json`` (schema v7), kernels pinned by sha256 and a Hugging
Face safetensors checkpoint bound by tensor name. The engine holds no model code: the native core
verifies a manifest without a GPU, compiles each program to a flat launch list and replays it as a
CUDA graph; a host-side pool pages KV and per-sequence state slots; the Python layer generates
manifests, is the PyTorch fp32 oracle, and hosts the OpenAI-style server.
"""
from __future__ import annotations

__version__ = "0.1.0"

from . import _build as _build

_build.ensure_built()

from . import _native  # noqa: E402

__all__ = ["_native", "__version__"]
