"""CPU restatement of nano-vllm's attention path — TEST INFRASTRUCTURE, not product code.

What it restates (reference file:line):
  * store_kvcache      — nanovllm/layers/attention.py:10-39: cache row slot_mapping[i] of the
    flattened ``[num_slots, Hkv*D]`` plane receives key[i] / value[i].
  * Attention.forward  — nanovllm/layers/attention.py:58-79: store first, then either the
    varlen causal prefill (packed K/V, or the cache read through block_tables when a prefix
    was cached) or the paged decode.
The attention arithmetic itself lives in the third-party flash-attn wheel (declared unpinned
in the reference's pyproject.toml:18; 2.8.3 in this image), which is not part of the
reference tree.  Its published semantics are restated here: fp32
``softmax(scale * Q K^T + mask) V`` with query head h reading KV head h // (Hq/Hkv), causal
mask aligned to the bottom-right corner (query i of Lq sees keys j <= i + Lk - Lq), rows with
no visible key giving zeros, paged K/V ``[num_blocks, 256, Hkv, D]`` addressed through an
int32 block table.  Arithmetic: bf16 inputs upcast to fp32,
``torch.nn.functional.scaled_dot_product_attention`` on the host.

Pinning: the reference has no tests or golden vectors for this path.  The oracle is pinned
by tests/golden/*.npz, which hold outputs of the reference's own ``Attention.forward`` and
``store_kvcache`` (Triton + flash-attn) recorded on a B200 by tests/golden/make_golden.py;
tests/test_oracle_golden.py checks this file against them.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

BLOCK_SIZE = 256


def store_kvcache_ref(key, value, k_cache, v_cache, slot_mapping):
    """In-place scatter on CPU tensors; rows with a negative slot are skipped (the Triton
    kernel of the reference has no such rows; the runner never emits them)."""
    n = key.shape[0]
    if n == 0 or k_cache.numel() == 0:
        return
    row = key.shape[1] * key.shape[2]
    slots = slot_mapping.to(torch.int64)
    keep = slots >= 0
    kf = k_cache.view(-1, row)
    vf = v_cache.view(-1, row)
    kf[slots[keep]] = key.reshape(n, row)[keep]
    vf[slots[keep]] = value.reshape(n, row)[keep]


def gather_paged(cache, block_table_row, length):
    """[length, Hkv, D] view of one sequence's tokens, in order, through its block table."""
    nblk = (length + BLOCK_SIZE - 1) // BLOCK_SIZE
    ids = block_table_row[:nblk].to(torch.int64)
    return cache[ids].reshape(nblk * BLOCK_SIZE, cache.shape[2], cache.shape[3])[:length]


def _sdpa(q, k, v, scale, mask=None):
    # q [Lq,Hq,D], k/v [Lk,Hkv,D] -> [Lq,Hq,D], fp32
    qf = q.float().transpose(0, 1).unsqueeze(0)
    kf = k.float().transpose(0, 1).unsqueeze(0)
    vf = v.float().transpose(0, 1).unsqueeze(0)
    o = F.scaled_dot_product_attention(qf, kf, vf, attn_mask=mask, scale=scale, enable_gqa=True)
    return o.squeeze(0).transpose(0, 1)


def decode_ref(q, k_cache, v_cache, context_lens, block_tables, scale):
    """q [B,Hq,D] -> fp32 [B,Hq,D]; sequences with context_len 0 give zeros."""
    B = q.shape[0]
    out = torch.zeros(q.shape, dtype=torch.float32)
    for b in range(B):
        n = int(context_lens[b])
        if n <= 0:
            continue
        k = gather_paged(k_cache, block_tables[b], n)
        v = gather_paged(v_cache, block_tables[b], n)
        out[b] = _sdpa(q[b:b + 1], k, v, scale)[0]
    return out


def prefill_ref(q, k, v, cu_seqlens_q, cu_seqlens_k, scale, block_tables=None):
    """q [sum Lq,Hq,D] -> fp32 [sum Lq,Hq,D].  ``k``/``v`` are packed rows
    ``[sum Lk,Hkv,D]`` when block_tables is None, else the cache planes."""
    out = torch.zeros(q.shape, dtype=torch.float32)
    B = cu_seqlens_q.numel() - 1
    for b in range(B):
        q0, q1 = int(cu_seqlens_q[b]), int(cu_seqlens_q[b + 1])
        k0, k1 = int(cu_seqlens_k[b]), int(cu_seqlens_k[b + 1])
        lq, lk = q1 - q0, k1 - k0
        if lq == 0:
            continue
        if block_tables is None:
            kb, vb = k[k0:k1], v[k0:k1]
        else:
            kb, vb = gather_paged(k, block_tables[b], lk), gather_paged(v, block_tables[b], lk)
        i = torch.arange(lq).unsqueeze(1)
        j = torch.arange(lk).unsqueeze(0)
        mask = j <= i + (lk - lq)
        o = _sdpa(q[q0:q1], kb, vb, scale, mask)
        dead = ~mask.any(dim=1)  # rows that see no key: zeros, not NaN
        if dead.any():
            o[dead] = 0.0
        out[q0:q1] = o
    return out


def attention_forward_ref(q, k, v, k_cache, v_cache, ctx, scale):
    """Whole layer on CPU tensors, same control flow as nanovllm/layers/attention.py:58-79.
    ``ctx`` carries is_prefill, cu_seqlens_q/k, slot_mapping, context_lens, block_tables.
    Mutates the caches; returns fp32 ``[N, Hq, D]``."""
    if k_cache.numel() and v_cache.numel():
        store_kvcache_ref(k, v, k_cache, v_cache, ctx.slot_mapping)
    if ctx.is_prefill:
        if ctx.block_tables is not None:
            return prefill_ref(q, k_cache, v_cache, ctx.cu_seqlens_q, ctx.cu_seqlens_k, scale, ctx.block_tables)
        return prefill_ref(q, k, v, ctx.cu_seqlens_q, ctx.cu_seqlens_k, scale)
    return decode_ref(q, k_cache, v_cache, ctx.context_lens, ctx.block_tables, scale)


# ---- pre-attention step (q/k RMSNorm + rotary embedding) ------------------------------------

def rms_norm_ref(x, weight, eps):
    """nanovllm/layers/layernorm.py:17-27 (RMSNorm.rms_forward) with its roundings: fp32
    normalisation, cast to the input dtype, then the multiply by the weight in that dtype."""
    orig = x.dtype
    xf = x.to(torch.float32)
    var = xf.pow(2).mean(dim=-1, keepdim=True)
    xf = xf * torch.rsqrt(var + eps)
    return xf.to(orig) * weight


def rotary_cache_ref(head_dim, max_position, base):
    """nanovllm/layers/rotary_embedding.py:28-37: [max_position, head_dim] fp32, cos then sin."""
    inv_freq = 1.0 / (base ** (torch.arange(0, head_dim, 2, dtype=torch.float) / head_dim))
    t = torch.arange(max_position, dtype=torch.float)
    freqs = torch.einsum("i,j -> ij", t, inv_freq)
    return torch.cat((freqs.cos(), freqs.sin()), dim=-1)


def apply_rotary_ref(x, cos, sin):
    """nanovllm/layers/rotary_embedding.py:6-16 (NeoX style: the two halves of a head rotate)."""
    cos, sin = cos.unsqueeze(-2), sin.unsqueeze(-2)
    x1, x2 = torch.chunk(x.to(torch.float32), 2, dim=-1)
    return torch.cat((x1 * cos - x2 * sin, x2 * cos + x1 * sin), dim=-1).to(x.dtype)


def qk_norm_rope_ref(qkv, positions, q_weight, k_weight, cos_sin_cache, eps, hq, hkv, d):
    """The q/k path of nanovllm/models/qwen3.py:89-105 (weights None: qwen2.py:87-90) on a CPU
    copy of the fused qkv activation.  Returns (q [N,hq,d], k [N,hkv,d], v [N,hkv,d])."""
    n = qkv.shape[0]
    q, k, v = qkv.split([hq * d, hkv * d, hkv * d], dim=-1)
    q, k, v = q.reshape(n, hq, d), k.reshape(n, hkv, d), v.reshape(n, hkv, d)
    if q_weight is not None:
        q, k = rms_norm_ref(q, q_weight, eps), rms_norm_ref(k, k_weight, eps)
    cos, sin = cos_sin_cache[positions].chunk(2, dim=-1)
    return apply_rotary_ref(q, cos, sin), apply_rotary_ref(k, cos, sin), v


# ---- sampling (nanovllm/layers/sampler.py:10-26) ------------------------------------------

def sampler_scores_ref(logits, temperatures, noise):
    """Per-row scores whose argmax is the token: the fp32 logits for a greedy row
    (temperature 0), softmax(logits / T) / (noise + 1e-10) for a sampled row, where ``noise``
    is the row's Exponential(1) draw (sampler.py:15-25)."""
    x = logits.to(torch.float32)
    t = temperatures.to(torch.float32)
    probs = torch.softmax(x / t.unsqueeze(1), dim=-1, dtype=torch.float32)
    race = probs / (noise.to(torch.float32) + 1e-10)
    return torch.where((t == 0).unsqueeze(1), x, race)


def sampler_ref(logits, temperatures, noise):
    """Tokens of Sampler.forward for a given exponential draw (sampler.py:26)."""
    return sampler_scores_ref(logits, temperatures, noise).argmax(dim=-1)


# ---- LM head + sampler under tensor parallelism (embed_head.py:68-88, sampler.py:10-26) -------

def lm_head_sample_ref(hidden, weight_shards, cu_seqlens_q, temperatures, noise):
    """Tokens of ``ParallelLMHead.forward`` followed by ``Sampler.forward``.  ``hidden`` [N, H];
    ``weight_shards``: one [V / ranks, H] matrix per rank, in rank order.  Under prefill
    (``cu_seqlens_q`` given) only each sequence's last row is kept (embed_head.py:72-74); every rank
    multiplies by its shard (:77), rank 0 concatenates the ranks' logits along the vocabulary
    (:78-87); the sampler then decides on the full rows with the given exponential draw."""
    x = hidden
    if cu_seqlens_q is not None:
        x = x[(cu_seqlens_q[1:] - 1).to(torch.int64)].contiguous()
    logits = torch.cat([F.linear(x, w) for w in weight_shards], dim=-1)
    return sampler_ref(logits, temperatures, noise), logits


def sample_candidates_ref(logits_slice, temperatures, noise_slice, vocab_offset):
    """What one rank contributes to the vocabulary-sharded tail: for every row the best
    (score, global index) of its slice, packed into an int64 whose signed order is "higher score,
    then lower index" (score bits mapped order-preservingly into the high word, 2^32 - 1 - index in
    the low word).  The element-wise maximum over the ranks, unpacked with
    ``sample_unpack_ref``, is the token of ``sampler_ref`` on the concatenated logits."""
    # A score that does not depend on the slice: softmax(x / T) / (e + 1e-10) has the same argmax
    # as x / T - ln(e + 1e-10), the softmax maximum and normaliser being constants of the whole row.
    x = logits_slice.to(torch.float32)
    t = temperatures.to(torch.float32).unsqueeze(1)
    race = x / t - torch.log(noise_slice.to(torch.float32) + 1e-10)
    scores = torch.where(t == 0, x, race)
    best = scores.max(dim=-1)
    bits = best.values.contiguous().view(torch.int32).to(torch.int64)
    ordered = torch.where(bits >= 0, bits, bits ^ 0x7FFFFFFF)
    # ties inside the slice: torch.max returns the first maximal index on the CPU
    idx = best.indices.to(torch.int64) + int(vocab_offset)
    return (ordered << 32) | (0xFFFFFFFF - idx)


def sample_unpack_ref(packed):
    return 0xFFFFFFFF - (packed & 0xFFFFFFFF)


# ---- decode-step inputs (nanovllm/engine/model_runner.py:151-159, 218-249, 271-282) ---------

def decode_inputs_ref(seqs, graph_bs, table_width, block_size=BLOCK_SIZE):
    """Rows [0, graph_bs) of the graph's static input tensors after the reference has prepared a
    decode step of ``seqs`` (objects with last_token, num_tokens, block_table) and refreshed the
    buffers: cleared, then the first len(seqs) rows overwritten, the block tables as a
    [bs, widest] tensor padded with -1."""
    import numpy as np
    n = len(seqs)
    out = {"input_ids": np.zeros(graph_bs, np.int64), "positions": np.zeros(graph_bs, np.int64),
           "slot_mapping": np.zeros(graph_bs, np.int32), "context_lens": np.zeros(graph_bs, np.int32),
           "block_tables": np.zeros((graph_bs, table_width), np.int32)}
    widest = max(len(s.block_table) for s in seqs)
    for i, s in enumerate(seqs):
        length = s.num_tokens
        num_blocks = (length + block_size - 1) // block_size
        last_block_tokens = length - (num_blocks - 1) * block_size
        out["input_ids"][i] = s.last_token
        out["positions"][i] = length
        out["context_lens"][i] = length
        out["slot_mapping"][i] = s.block_table[-1] * block_size + last_block_tokens - 1
        row = list(s.block_table) + [-1] * (widest - len(s.block_table))
        out["block_tables"][i, :widest] = row
    assert n <= graph_bs
    return out


# ---- tensor-parallel sum (nanovllm/layers/linear.py:195-199) --------------------------------

def allreduce_ref(inputs):
    """Sum of the ranks' bf16 tensors: fp32 accumulation in rank order, rounded to bf16 once."""
    acc = torch.zeros(inputs[0].shape, dtype=torch.float32)
    for x in inputs:
        acc += x.to(torch.float32)
    return acc.to(torch.bfloat16)


def row_parallel_linear_ref(xs, weights):
    """RowParallelLinear.forward over all ranks (nanovllm/layers/linear.py:195-199, no bias):
    every rank's F.linear in fp32 rounded to bf16 (what the rank's GEMM returns), then the sum of
    those partials as ``allreduce_ref`` forms it."""
    partials = [(x.to(torch.float32) @ w.to(torch.float32).t()).to(torch.bfloat16) for x, w in zip(xs, weights)]
    return allreduce_ref(partials)
