"""Attention layer of nano-vllm on the B200 kernels: the host side of the C ABI.

Same surface as nanovllm/layers/attention.py:32-79 — ``store_kvcache(key, value, k_cache,
v_cache, slot_mapping)`` and ``Attention(num_heads, head_dim, scale, num_kv_heads)`` with the
``k_cache`` / ``v_cache`` attributes that the model runner binds
(nanovllm/engine/model_runner.py:145-149) and ``forward(q, k, v)`` driven by the per-step
context — but every device operation goes through libnvllm_b200.so.  Tensors must live on a
CUDA device and be bf16; anything else raises (there is no CPU or eager fallback).
"""
from __future__ import annotations

from typing import Callable

import torch
from torch import nn

from . import _lib
from . import context as _own_context

BLOCK_SIZE = 256

_get_context: Callable[[], object] = _own_context.get_context


def use_context_getter(getter: Callable[[], object]) -> None:
    """Makes ``Attention.forward`` read its metadata from another module's ``get_context``
    (nano-vllm's ``nanovllm.utils.context.get_context`` when running inside that engine)."""
    global _get_context
    _get_context = getter


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _require_cuda_bf16(name: str, t: torch.Tensor) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor (nano_vllm_b200 has no CPU path)")
    if t.dtype != torch.bfloat16:
        raise RuntimeError(f"{name} must be bfloat16, got {t.dtype}")


def _require_i32(name: str, t: torch.Tensor) -> None:
    if not t.is_cuda or t.dtype != torch.int32 or (t.dim() > 0 and t.stride(-1) != 1):
        raise RuntimeError(f"{name} must be a CUDA int32 tensor with unit inner stride")


# ---- decode scratch ---------------------------------------------------------------------
# One buffer per device, grown on demand and zero-filled when it is made: its head holds the
# arrival counters of the decode kernel, which must start at zero and which every completed
# call leaves at zero.  Outgrown buffers are kept alive because CUDA graphs captured earlier
# still hold their addresses.
_workspaces: dict[int, torch.Tensor] = {}
_retired: list[torch.Tensor] = []


def _workspace(device: torch.device, nbytes: int) -> torch.Tensor | None:
    if nbytes == 0:
        return None
    idx = device.index if device.index is not None else torch.cuda.current_device()
    ws = _workspaces.get(idx)
    if ws is None or ws.numel() < nbytes:
        if ws is not None:
            _retired.append(ws)
        ws = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[idx] = ws
    return ws


# ---- functional entry points ------------------------------------------------------------

def store_kvcache(key: torch.Tensor, value: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                  slot_mapping: torch.Tensor) -> None:
    """k_cache.view(-1, Hkv*D)[slot_mapping[i]] = key[i] (same for value); bit-exact copy.

    Same argument contract and asserts as nanovllm/layers/attention.py:32-39.
    """
    N, num_heads, head_dim = key.shape
    D = num_heads * head_dim
    assert key.stride(-1) == 1 and value.stride(-1) == 1
    assert key.stride(1) == head_dim and value.stride(1) == head_dim
    assert k_cache.stride(1) == D and v_cache.stride(1) == D
    assert slot_mapping.numel() == N
    for name, t in (("key", key), ("value", value), ("k_cache", k_cache), ("v_cache", v_cache)):
        _require_cuda_bf16(name, t)
    _require_i32("slot_mapping", slot_mapping)
    num_slots = k_cache.numel() // D
    with torch.cuda.device(key.device):
        _lib.check(_lib.load().nvllm_store_kvcache(
            key.data_ptr(), key.stride(0), value.data_ptr(), value.stride(0),
            k_cache.data_ptr(), v_cache.data_ptr(), slot_mapping.data_ptr(),
            N, D, num_slots, _stream(key)))


def decode_paged(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, context_lens: torch.Tensor,
                 block_tables: torch.Tensor, scale: float, out: torch.Tensor | None = None) -> torch.Tensor:
    """One query token per sequence against the paged cache; q/out are ``[B, Hq, D]``.

    Stands where ``flash_attn_with_kvcache(q.unsqueeze(1), k_cache, v_cache,
    cache_seqlens=context_lens, block_table=block_tables, softmax_scale=scale, causal=True)``
    stands in nanovllm/layers/attention.py:74-77.
    """
    B, Hq, D = q.shape
    Hkv = k_cache.shape[-2]
    _require_cuda_bf16("q", q)
    _require_cuda_bf16("k_cache", k_cache)
    _require_cuda_bf16("v_cache", v_cache)
    _require_i32("context_lens", context_lens)
    _require_i32("block_tables", block_tables)
    assert q.stride(-1) == 1 and q.stride(1) == D
    assert k_cache.is_contiguous() and v_cache.is_contiguous()
    assert block_tables.dim() == 2 and block_tables.shape[0] == B and context_lens.numel() == B
    if out is None:
        out = torch.empty((B, Hq, D), dtype=q.dtype, device=q.device)
    assert out.stride(-1) == 1 and out.stride(1) == D
    max_blocks = block_tables.shape[1]
    num_blocks = k_cache.numel() // (BLOCK_SIZE * Hkv * D)
    if B == 0:
        return out
    with torch.cuda.device(q.device):
        ws = _workspace(q.device, _lib.decode_workspace_bytes(B, max_blocks, Hq, Hkv, D))
        _lib.check(_lib.load().nvllm_decode_paged(
            q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(),
            context_lens.data_ptr(), block_tables.data_ptr(), block_tables.stride(0), max_blocks,
            out.data_ptr(), out.stride(0), B, Hq, Hkv, D, float(scale), num_blocks,
            ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0, _stream(q)))
    return out


def decode_step(q: torch.Tensor, key: torch.Tensor, value: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                slot_mapping: torch.Tensor, context_lens: torch.Tensor, block_tables: torch.Tensor, scale: float,
                out: torch.Tensor | None = None) -> torch.Tensor:
    """``store_kvcache(key, value, k_cache, v_cache, slot_mapping)`` followed by ``decode_paged`` as
    ONE launch: what nanovllm/layers/attention.py:65-66 and :74-77 do for a decode batch.  The
    thread block that streams a sequence's newest position takes that row from ``key`` /
    ``value`` and writes it to the cache on the way.  ``slot_mapping[b]`` must be the slot of
    position ``context_lens[b] - 1`` (what the model runner passes) or negative (nothing stored);
    rows with ``context_lens[b] == 0`` store nothing.  q/out ``[B, Hq, D]``, key/value ``[B, Hkv, D]``.
    """
    B, Hq, D = q.shape
    Hkv = k_cache.shape[-2]
    for name, t in (("q", q), ("key", key), ("value", value), ("k_cache", k_cache), ("v_cache", v_cache)):
        _require_cuda_bf16(name, t)
    _require_i32("slot_mapping", slot_mapping)
    _require_i32("context_lens", context_lens)
    _require_i32("block_tables", block_tables)
    assert q.stride(-1) == 1 and q.stride(1) == D
    assert key.shape == (B, Hkv, D) and value.shape == (B, Hkv, D)
    assert key.stride(-1) == 1 and value.stride(-1) == 1 and key.stride(1) == D and value.stride(1) == D
    assert k_cache.is_contiguous() and v_cache.is_contiguous()
    assert block_tables.dim() == 2 and block_tables.shape[0] == B and context_lens.numel() == B
    assert slot_mapping.numel() == B
    if out is None:
        out = torch.empty((B, Hq, D), dtype=q.dtype, device=q.device)
    assert out.stride(-1) == 1 and out.stride(1) == D
    max_blocks = block_tables.shape[1]
    num_blocks = k_cache.numel() // (BLOCK_SIZE * Hkv * D)
    if B == 0:
        return out
    with torch.cuda.device(q.device):
        ws = _workspace(q.device, _lib.decode_workspace_bytes(B, max_blocks, Hq, Hkv, D))
        _lib.check(_lib.load().nvllm_decode_step(
            q.data_ptr(), q.stride(0), key.data_ptr(), key.stride(0), value.data_ptr(), value.stride(0),
            slot_mapping.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
            context_lens.data_ptr(), block_tables.data_ptr(), block_tables.stride(0), max_blocks,
            out.data_ptr(), out.stride(0), B, Hq, Hkv, D, float(scale), num_blocks,
            ws.data_ptr(), ws.numel(), _stream(q)))
    return out


def decode_paged_static(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, context_lens: torch.Tensor,
                        block_tables: torch.Tensor, scale: float, out: torch.Tensor) -> torch.Tensor:
    """``decode_paged`` for hosts that may not allocate device memory while serving (all free
    HBM already belongs to the KV cache, or an allocation's implicit synchronisation is not
    acceptable): the arrival counters and partials go to a 32 MiB array inside the library instead
    of a torch-allocated workspace, and ``out`` must be supplied, so this call allocates nothing.
    Raises ``NvllmError`` (NVLLM_E_WORKSPACE) for geometries whose scratch exceeds the array.
    Calls on one device share that array: keep them ordered on the GPU.  Make the first call
    on a device outside CUDA graph capture.  No counterpart in nano-vllm."""
    B, Hq, D = q.shape
    Hkv = k_cache.shape[-2]
    _require_cuda_bf16("q", q)
    _require_cuda_bf16("k_cache", k_cache)
    _require_cuda_bf16("v_cache", v_cache)
    _require_cuda_bf16("out", out)
    _require_i32("context_lens", context_lens)
    _require_i32("block_tables", block_tables)
    assert q.stride(-1) == 1 and q.stride(1) == D and out.stride(-1) == 1 and out.stride(1) == D
    assert k_cache.is_contiguous() and v_cache.is_contiguous()
    assert block_tables.dim() == 2 and block_tables.shape[0] == B and context_lens.numel() == B
    num_blocks = k_cache.numel() // (BLOCK_SIZE * Hkv * D)
    with torch.cuda.device(q.device):
        _lib.check(_lib.load().nvllm_decode_paged_static(
            q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(),
            context_lens.data_ptr(), block_tables.data_ptr(), block_tables.stride(0), block_tables.shape[1],
            out.data_ptr(), out.stride(0), B, Hq, Hkv, D, float(scale), num_blocks, _stream(q)))
    return out


def prefill_varlen(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens_q: torch.Tensor,
                   cu_seqlens_k: torch.Tensor, max_seqlen_q: int, max_seqlen_k: int, scale: float,
                   block_tables: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """Varlen causal GQA attention over packed K/V rows, or over the paged cache when
    ``block_tables`` is given (then ``k``/``v`` are the cache planes).  q/out: ``[N, Hq, D]``.

    Stands where ``flash_attn_varlen_func(..., causal=True, block_table=block_tables)`` stands
    in nanovllm/layers/attention.py:70-73.
    """
    N, Hq, D = q.shape
    Hkv = k.shape[-2]
    for name, t in (("q", q), ("k", k), ("v", v)):
        _require_cuda_bf16(name, t)
    _require_i32("cu_seqlens_q", cu_seqlens_q)
    _require_i32("cu_seqlens_k", cu_seqlens_k)
    assert q.stride(-1) == 1 and q.stride(1) == D
    batch = cu_seqlens_q.numel() - 1
    assert cu_seqlens_k.numel() == batch + 1
    if out is None:
        out = torch.empty((N, Hq, D), dtype=q.dtype, device=q.device)
    assert out.stride(-1) == 1 and out.stride(1) == D
    if block_tables is not None:
        _require_i32("block_tables", block_tables)
        assert k.is_contiguous() and v.is_contiguous() and k.dim() == 4 and k.shape[1] == BLOCK_SIZE
        assert block_tables.dim() == 2 and block_tables.shape[0] == batch
        bt_ptr, bt_stride, max_blocks = block_tables.data_ptr(), block_tables.stride(0), block_tables.shape[1]
        num_blocks = k.shape[0]
        k_stride = v_stride = Hkv * D
    else:
        assert k.dim() == 3 and k.stride(-1) == 1 and v.stride(-1) == 1 and k.stride(1) == D and v.stride(1) == D
        bt_ptr, bt_stride, max_blocks, num_blocks = None, 0, 0, 0
        k_stride, v_stride = k.stride(0), v.stride(0)
    if N == 0 or batch == 0:
        return out
    with torch.cuda.device(q.device):
        _lib.check(_lib.load().nvllm_prefill_varlen(
            q.data_ptr(), q.stride(0), k.data_ptr(), k_stride, v.data_ptr(), v_stride,
            bt_ptr, bt_stride, max_blocks, out.data_ptr(), out.stride(0),
            cu_seqlens_q.data_ptr(), cu_seqlens_k.data_ptr(), N, 0 if block_tables is not None else k.shape[0],
            batch, int(max_seqlen_q), int(max_seqlen_k),
            Hq, Hkv, D, float(scale), num_blocks, _stream(q)))
    return out


def qk_norm_rope_store(qkv: torch.Tensor, positions: torch.Tensor, q_weight: torch.Tensor | None,
                       k_weight: torch.Tensor | None, cos_sin_cache: torch.Tensor, eps: float,
                       slot_mapping: torch.Tensor | None, k_cache: torch.Tensor, v_cache: torch.Tensor,
                       num_q_heads: int, num_kv_heads: int, head_dim: int) -> None:
    """In place on the fused ``qkv`` activation ``[N, (Hq + 2*Hkv) * D]``: per-head RMSNorm of
    q and k (when weights are given), rotary embedding of q and k, and the scatter of the new
    K/V rows into the cache (when ``slot_mapping`` is given and the cache exists).

    One launch for what nanovllm/models/qwen3.py:89-107 does with ``q_norm``, ``k_norm``,
    ``rotary_emb`` and, inside the attention layer, ``store_kvcache``.
    """
    _require_cuda_bf16("qkv", qkv)
    assert qkv.dim() == 2 and qkv.stride(-1) == 1
    assert qkv.shape[1] == (num_q_heads + 2 * num_kv_heads) * head_dim
    assert positions.is_cuda and positions.dtype == torch.int64 and positions.numel() == qkv.shape[0]
    assert cos_sin_cache.is_cuda and cos_sin_cache.dtype == torch.float32 and cos_sin_cache.is_contiguous()
    cs = cos_sin_cache.view(-1, head_dim)
    for w in (q_weight, k_weight):
        if w is not None:
            _require_cuda_bf16("norm weight", w)
            assert w.numel() == head_dim and w.is_contiguous()
    store = slot_mapping is not None and k_cache.numel() > 0 and v_cache.numel() > 0
    if store:
        _require_i32("slot_mapping", slot_mapping)
        _require_cuda_bf16("k_cache", k_cache)
        _require_cuda_bf16("v_cache", v_cache)
        assert k_cache.is_contiguous() and v_cache.is_contiguous() and slot_mapping.numel() == qkv.shape[0]
    num_slots = k_cache.numel() // (num_kv_heads * head_dim) if store else 0
    with torch.cuda.device(qkv.device):
        _lib.check(_lib.load().nvllm_qk_norm_rope_store(
            qkv.data_ptr(), qkv.stride(0), positions.data_ptr(),
            q_weight.data_ptr() if q_weight is not None else None,
            k_weight.data_ptr() if k_weight is not None else None,
            cs.data_ptr(), cs.shape[0], float(eps),
            slot_mapping.data_ptr() if store else None,
            k_cache.data_ptr() if store else None, v_cache.data_ptr() if store else None, num_slots,
            qkv.shape[0], num_q_heads, num_kv_heads, head_dim, _stream(qkv)))


def sample_tokens(logits: torch.Tensor, temperatures: torch.Tensor, noise: torch.Tensor | None = None,
                  seed: int = 0, step: int = 0, out: torch.Tensor | None = None) -> torch.Tensor:
    """One token per row of ``logits`` ``[B, V]`` (bf16 or fp32): argmax where the row's temperature
    is 0, else a draw from ``softmax(logits / T)``.  One launch for what
    nanovllm/layers/sampler.py:10-26 does in eight.  ``noise`` ``[B, V]`` fp32, when given, is the
    Exponential(1) draw to use (the reference's ``torch.empty_like(probs).exponential_(1)``);
    otherwise the kernel generates its own from ``(seed, step)``.  Returns int64 ``[B]``.
    """
    assert logits.is_cuda and logits.dim() == 2 and logits.stride(-1) == 1
    assert logits.dtype in (torch.bfloat16, torch.float32), f"logits must be bf16 or fp32, got {logits.dtype}"
    B, V = logits.shape
    assert temperatures.is_cuda and temperatures.dtype == torch.float32 and temperatures.numel() == B
    assert temperatures.is_contiguous()
    if noise is not None:
        assert noise.is_cuda and noise.dtype == torch.float32 and noise.shape == logits.shape and noise.stride(-1) == 1
    if out is None:
        out = torch.empty(B, dtype=torch.int64, device=logits.device)
    else:
        assert out.is_cuda and out.dtype == torch.int64 and out.numel() == B and out.is_contiguous()
    with torch.cuda.device(logits.device):
        _lib.check(_lib.load().nvllm_sample_tokens(
            logits.data_ptr(), 1 if logits.dtype == torch.float32 else 0, logits.stride(0), temperatures.data_ptr(),
            noise.data_ptr() if noise is not None else None, noise.stride(0) if noise is not None else 0,
            seed & 0xFFFFFFFFFFFFFFFF, step & 0xFFFFFFFFFFFFFFFF, out.data_ptr(), B, V, _stream(logits)))
    return out


def sample_candidates(logits: torch.Tensor, temperatures: torch.Tensor, vocab_offset: int, noise: torch.Tensor | None = None,
                      seed: int = 0, step: int = 0, out: torch.Tensor | None = None) -> torch.Tensor:
    """``sample_tokens`` for one rank's slice ``[B, V / ranks]`` of the vocabulary, starting at global
    index ``vocab_offset``: returns int64 ``[B]`` candidates whose element-wise maximum over the ranks
    (``dist.reduce(..., op=MAX)``) decodes, with ``sample_unpack``, to the token ``sample_tokens``
    picks from the concatenated logits.  Replaces the gather + cat of
    nanovllm/layers/embed_head.py:78-87 by 8 bytes per row."""
    assert logits.is_cuda and logits.dim() == 2 and logits.stride(-1) == 1
    assert logits.dtype in (torch.bfloat16, torch.float32), f"logits must be bf16 or fp32, got {logits.dtype}"
    B, V = logits.shape
    assert temperatures.is_cuda and temperatures.dtype == torch.float32 and temperatures.numel() == B
    assert temperatures.is_contiguous()
    if noise is not None:
        assert noise.is_cuda and noise.dtype == torch.float32 and noise.shape == logits.shape and noise.stride(-1) == 1
    if out is None:
        out = torch.empty(B, dtype=torch.int64, device=logits.device)
    else:
        assert out.is_cuda and out.dtype == torch.int64 and out.numel() == B and out.is_contiguous()
    with torch.cuda.device(logits.device):
        _lib.check(_lib.load().nvllm_sample_candidates(
            logits.data_ptr(), 1 if logits.dtype == torch.float32 else 0, logits.stride(0), temperatures.data_ptr(),
            noise.data_ptr() if noise is not None else None, noise.stride(0) if noise is not None else 0,
            seed & 0xFFFFFFFFFFFFFFFF, step & 0xFFFFFFFFFFFFFFFF, int(vocab_offset), out.data_ptr(), B, V, _stream(logits)))
    return out


def sample_unpack(candidates: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """Token ids int64 ``[B]`` of (merged) candidates from ``sample_candidates``."""
    assert candidates.is_cuda and candidates.dtype == torch.int64 and candidates.is_contiguous()
    B = candidates.numel()
    if out is None:
        out = torch.empty(B, dtype=torch.int64, device=candidates.device)
    with torch.cuda.device(candidates.device):
        _lib.check(_lib.load().nvllm_sample_unpack(candidates.data_ptr(), out.data_ptr(), B, _stream(candidates)))
    return out


# ---- the layer --------------------------------------------------------------------------

class Attention(nn.Module):
    """Drop-in for nanovllm/layers/attention.py:42-79 (same constructor, attributes, forward)."""

    def __init__(self, num_heads, head_dim, scale, num_kv_heads):
        super().__init__()
        self.num_heads = num_heads
        self.head_dim = head_dim
        self.scale = scale
        self.num_kv_heads = num_kv_heads
        self.k_cache = self.v_cache = torch.tensor([])

    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, kv_stored: bool = False):
        """``kv_stored=True``: the caller has already written this step's K/V rows into the cache
        (the fused pre-attention step does); the reference signature is ``forward(q, k, v)``."""
        q = q.view(-1, self.num_heads, self.head_dim)
        k = k.view(-1, self.num_kv_heads, self.head_dim)
        v = v.view(-1, self.num_kv_heads, self.head_dim)
        context = _get_context()
        k_cache, v_cache = self.k_cache, self.v_cache
        if k_cache.numel() and v_cache.numel() and not kv_stored:
            store_kvcache(k, v, k_cache, v_cache, context.slot_mapping)
        if context.is_prefill:
            if context.block_tables is not None:  # prefix cache: read every key through the table
                k, v = k_cache, v_cache
            o = prefill_varlen(q, k, v, context.cu_seqlens_q, context.cu_seqlens_k,
                               context.max_seqlen_q, context.max_seqlen_k, self.scale,
                               block_tables=context.block_tables)
        else:
            o = decode_paged(q, k_cache, v_cache, context.context_lens, context.block_tables, self.scale)
        return o.view(-1, self.num_heads * self.head_dim)
