"""Installs the B200 attention layer into an importable nano-vllm without editing its tree.

``install()`` registers a module named ``nanovllm.layers.attention`` that exports the same two
names the reference module exports (``Attention``, ``store_kvcache``;
nanovllm/layers/attention.py:32-79) and makes the layer read nano-vllm's own per-step context
(nanovllm/utils/context.py:16-17).  Call it before ``nanovllm.models`` is imported (i.e. before
``from nanovllm import LLM``), because the model files bind ``Attention`` at import time
(nanovllm/models/qwen3.py:8).
"""
from __future__ import annotations

import importlib
import sys
import types

from . import attention as _attention

MODULE_NAME = "nanovllm.layers.attention"


def install() -> types.ModuleType:
    late = [m for m in ("nanovllm.models.qwen3", "nanovllm.models.qwen2") if m in sys.modules]
    if late and getattr(sys.modules.get(MODULE_NAME), "__nano_vllm_b200__", False) is False:
        raise RuntimeError(f"install() must run before {late[0]} is imported")
    ctx = importlib.import_module("nanovllm.utils.context")
    _attention.use_context_getter(ctx.get_context)
    mod = types.ModuleType(MODULE_NAME)
    mod.__doc__ = "nano-vllm attention layer backed by libnvllm_b200.so"
    mod.Attention = _attention.Attention
    mod.store_kvcache = _attention.store_kvcache
    mod.get_context = ctx.get_context
    mod.__nano_vllm_b200__ = True
    sys.modules[MODULE_NAME] = mod
    layers = sys.modules.get("nanovllm.layers")
    if layers is not None:
        setattr(layers, "attention", mod)
    return mod
