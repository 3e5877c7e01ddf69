"""Seeded synthetic inputs for the attention path, shaped like what nano-vllm's model runner
hands to the attention layer (nanovllm/engine/model_runner.py:151-249), plus the
algorithmic work (bytes / flops) of each case.

The reference measures on random token ids (its bench.py:9-28 draws lengths with
``randint(100, 1024)``); there is no dataset to stand in for.  Everything here is generated
from ``torch.Generator().manual_seed(seed)`` so the CUDA path and the CPU oracle see the
same values.
"""
from __future__ import annotations

from dataclasses import dataclass, fields

import torch

BLOCK_SIZE = 256


def _blocks(n_tokens: int) -> int:
    return (n_tokens + BLOCK_SIZE - 1) // BLOCK_SIZE


class _Case:
    def to(self, device):
        """Copy of the case with every tensor moved to ``device``."""
        kw = {}
        for f in fields(self):
            val = getattr(self, f.name)
            kw[f.name] = val.to(device) if isinstance(val, torch.Tensor) else val
        return type(self)(**kw)


@dataclass
class DecodeCase(_Case):
    """One decode step of one layer: ``batch`` sequences, one new token each."""
    q: torch.Tensor             # [B, Hq, D] bf16
    k_new: torch.Tensor         # [B, Hkv, D] bf16, K of the token being decoded
    v_new: torch.Tensor         # [B, Hkv, D] bf16
    k_cache: torch.Tensor       # [num_blocks, 256, Hkv, D] bf16 (new token's slot not yet written)
    v_cache: torch.Tensor
    context_lens: torch.Tensor  # [B] int32, length including the new token
    block_tables: torch.Tensor  # [B, max_blocks] int32, -1 past a sequence's blocks
    slot_mapping: torch.Tensor  # [B] int32, slot of token context_len-1
    scale: float

    @property
    def geometry(self):
        B, Hq, D = self.q.shape
        return B, Hq, self.k_new.shape[1], D


@dataclass
class PrefillCase(_Case):
    """One prefill batch of one layer.  Sequence b has Lk_b tokens of which the last Lq_b are
    new; the first Lk_b - Lq_b (a multiple of 256) are a prefix-cache hit."""
    q: torch.Tensor             # [sum Lq, Hq, D] bf16
    k: torch.Tensor             # [sum Lq, Hkv, D] bf16 (new tokens only)
    v: torch.Tensor
    k_cache: torch.Tensor       # [num_blocks, 256, Hkv, D] bf16 (may be empty: no cache yet)
    v_cache: torch.Tensor
    cu_seqlens_q: torch.Tensor  # [B+1] int32
    cu_seqlens_k: torch.Tensor  # [B+1] int32
    max_seqlen_q: int
    max_seqlen_k: int
    slot_mapping: torch.Tensor  # [sum Lq] int32
    block_tables: torch.Tensor | None  # [B, max_blocks] int32 or None when nothing is cached
    scale: float


def _randn_bf16(shape, gen: torch.Generator, device) -> torch.Tensor:
    if torch.device(device).type == "cpu":
        return torch.randn(shape, generator=gen, dtype=torch.float32).to(torch.bfloat16)
    return torch.randn(shape, generator=gen, dtype=torch.bfloat16, device=device)


def make_decode_case(seed: int, batch: int, ctx_lo: int, ctx_hi: int, hq: int, hkv: int, d: int,
                     device="cpu", spare_blocks: int | None = None, table_width: int | None = None,
                     context_lens: list[int] | None = None) -> DecodeCase:
    """Context lengths uniform in [ctx_lo, ctx_hi] (or given), physical blocks a seeded random
    permutation of a pool with spare blocks, q/k/v ~ N(0,1) in bf16.  Metadata is drawn from a
    CPU generator; the big tensors from a generator on ``device``."""
    g = torch.Generator().manual_seed(seed)
    if context_lens is None:
        lens = torch.randint(ctx_lo, ctx_hi + 1, (batch,), generator=g)
    else:
        lens = torch.tensor(context_lens, dtype=torch.int64)
        assert lens.numel() == batch
    nblk = [(_blocks(int(n))) for n in lens]
    total = sum(nblk)
    spare = max(2, total // 8) if spare_blocks is None else spare_blocks
    num_blocks = total + spare
    perm = torch.randperm(num_blocks, generator=g)
    width = max(max(nblk), 1) if table_width is None else table_width
    assert width >= max(nblk + [0])
    bt = torch.full((batch, width), -1, dtype=torch.int32)
    slots = torch.zeros(batch, dtype=torch.int32)
    pos = 0
    for b in range(batch):
        ids = perm[pos:pos + nblk[b]].to(torch.int32)
        pos += nblk[b]
        bt[b, :nblk[b]] = ids
        n = int(lens[b])
        slots[b] = int(ids[-1]) * BLOCK_SIZE + (n - 1) % BLOCK_SIZE if n > 0 else -1
    gd = g if torch.device(device).type == "cpu" else torch.Generator(device=device).manual_seed(seed)
    q = _randn_bf16((batch, hq, d), gd, device)
    k_new = _randn_bf16((batch, hkv, d), gd, device)
    v_new = _randn_bf16((batch, hkv, d), gd, device)
    k_cache = _randn_bf16((num_blocks, BLOCK_SIZE, hkv, d), gd, device)
    v_cache = _randn_bf16((num_blocks, BLOCK_SIZE, hkv, d), gd, device)
    return DecodeCase(q, k_new, v_new, k_cache, v_cache, lens.to(torch.int32).to(device), bt.to(device),
                      slots.to(device), float(d) ** -0.5)


def make_prefill_case(seed: int, batch: int, len_lo: int, len_hi: int, hq: int, hkv: int, d: int,
                      device="cpu", share_every: int = 4, lengths: list[int] | None = None,
                      shared_blocks: list[int] | None = None, with_cache: bool = True,
                      spare_blocks: int = 3) -> PrefillCase:
    """Prompt lengths uniform in [len_lo, len_hi].  With ``share_every`` = n > 0, every sequence
    i with i % n == n-1 shares its first 1-3 blocks with sequence i-1 (same physical blocks,
    so its Lq < Lk), clipped so that at least one token stays uncached; ``shared_blocks`` gives
    the number of shared blocks per sequence explicitly.  ``with_cache=False`` models the
    engine's warm-up prefill (no cache allocated, no table)."""
    g = torch.Generator().manual_seed(seed)
    if lengths is None:
        lens = torch.randint(len_lo, len_hi + 1, (batch,), generator=g).tolist()
    else:
        lens = list(lengths)
        assert len(lens) == batch
    if shared_blocks is None:
        shared = [0] * batch
        if share_every > 0 and with_cache:
            want = torch.randint(1, 4, (batch,), generator=g).tolist()
            for i in range(batch):
                if i % share_every == share_every - 1 and i > 0 and shared[i - 1] == 0:
                    if min(lens[i], lens[i - 1]) <= BLOCK_SIZE:  # make one shareable block exist
                        lens[i] = max(lens[i], BLOCK_SIZE + 1)
                        lens[i - 1] = max(lens[i - 1], BLOCK_SIZE + 1)
                    s = min(want[i], (lens[i] - 1) // BLOCK_SIZE, lens[i - 1] // BLOCK_SIZE)
                    shared[i] = max(s, 0)
    else:
        shared = list(shared_blocks)
        for i, s_ in enumerate(shared):  # only whole blocks of the predecessor can be shared
            assert s_ == 0 or (i > 0 and s_ <= lens[i - 1] // BLOCK_SIZE and s_ * BLOCK_SIZE <= lens[i])
    cached = [s * BLOCK_SIZE for s in shared]
    lq = [lens[i] - cached[i] for i in range(batch)]
    assert all(x >= 0 for x in lq)
    cu_q = torch.tensor([0] + list(torch.tensor(lq).cumsum(0).tolist()), dtype=torch.int32)
    cu_k = torch.tensor([0] + list(torch.tensor(lens).cumsum(0).tolist()), dtype=torch.int32)
    nq = int(cu_q[-1])

    nblk = [_blocks(n) for n in lens]
    own = [nblk[i] - shared[i] for i in range(batch)]
    num_blocks = sum(own) + spare_blocks
    perm = torch.randperm(num_blocks, generator=g).tolist()
    width = max(nblk + [1])
    bt = torch.full((batch, width), -1, dtype=torch.int32)
    slot_list: list[int] = []
    pos = 0
    for i in range(batch):
        ids = (bt[i - 1, :shared[i]].tolist() if shared[i] else []) + perm[pos:pos + own[i]]
        pos += own[i]
        bt[i, :nblk[i]] = torch.tensor(ids, dtype=torch.int32)
        for t in range(cached[i], lens[i]):
            slot_list.append(ids[t // BLOCK_SIZE] * BLOCK_SIZE + t % BLOCK_SIZE)
    gd = g if torch.device(device).type == "cpu" else torch.Generator(device=device).manual_seed(seed)
    q = _randn_bf16((nq, hq, d), gd, device)
    k = _randn_bf16((nq, hkv, d), gd, device)
    v = _randn_bf16((nq, hkv, d), gd, device)
    if with_cache:
        k_cache = torch.zeros((num_blocks, BLOCK_SIZE, hkv, d), dtype=torch.bfloat16, device=device)
        v_cache = torch.zeros_like(k_cache)
        slot_mapping = torch.tensor(slot_list, dtype=torch.int32)
        block_tables = bt if any(shared) else None
    else:
        k_cache = torch.zeros(0, dtype=torch.bfloat16, device=device)
        v_cache = torch.zeros(0, dtype=torch.bfloat16, device=device)
        slot_mapping = torch.zeros(0, dtype=torch.int32)
        block_tables = None
    return PrefillCase(q, k, v, k_cache, v_cache, cu_q.to(device), cu_k.to(device), max(lq + [0]), max(lens + [0]),
                       slot_mapping.to(device), None if block_tables is None else block_tables.to(device),
                       float(d) ** -0.5)


# ---- the benchmark configurations ----------------------------------------------------------

QWEN3_06B = dict(hq=16, hkv=8, d=128)   # models/qwen3_06b.txt:10-20 of the reference
QWEN3_8B = dict(hq=32, hkv=8, d=128)
QWEN2_05B = dict(hq=14, hkv=2, d=64)    # models/qwen2_05b.txt:10-19


def cfg1_decode(device="cpu") -> DecodeCase:
    """8 sequences, contexts in [100,1024], Qwen3-0.6B geometry."""
    return make_decode_case(1, 8, 100, 1024, device=device, **QWEN3_06B)


def cfg2_prefill(device="cpu") -> PrefillCase:
    """64 prompts in [100,1024]; every 4th shares 1-3 blocks with its predecessor."""
    return make_prefill_case(2, 64, 100, 1024, device=device, **QWEN3_06B)


def cfg4_decode(tp: int = 1, rank: int = 0, device="cuda", batch: int = 256) -> DecodeCase:
    """Qwen3-8B geometry, batch 256, contexts in [2048,8192]; rank's head shard under TP=tp.
    Lengths and tables are identical on every rank (same seed); values differ per rank."""
    assert 8 % tp == 0
    case = make_decode_case(4, batch, 2048, 8192, hq=32 // tp, hkv=8 // tp, d=128, device=device,
                            spare_blocks=64)
    if rank:  # different values per shard, same metadata
        gd = torch.Generator(device=device).manual_seed(4000 + rank)
        case.q.copy_(_randn_bf16(tuple(case.q.shape), gd, device))
    return case


def cfg5_decode(tp: int = 1, device="cuda", batch: int = 512, ctx: int = 32768) -> DecodeCase:
    """Qwen2-0.5B geometry, every context 32768 tokens = 128 scattered blocks."""
    assert tp in (1, 2)
    return make_decode_case(5, batch, ctx, ctx, hq=14 // tp, hkv=2 // tp, d=64, device=device, spare_blocks=64)


# ---- algorithmic work ---------------------------------------------------------------------

def decode_bytes(context_lens, hq: int, hkv: int, d: int) -> int:
    """Bytes a decode step must move: every live K and V element once, q in, o out, lengths
    and the block-table entries in use.  Split-KV partials are overhead and not counted."""
    lens = [int(x) for x in context_lens]
    kv = sum(lens) * hkv * d * 2 * 2
    qo = 2 * len(lens) * hq * d * 2
    meta = 4 * (len(lens) + sum(_blocks(n) for n in lens))
    return kv + qo + meta


def store_bytes(n_tokens: int, row_elems: int) -> int:
    """K and V rows read once and written once, plus the slot ids."""
    return n_tokens * row_elems * 2 * 2 * 2 + 4 * n_tokens


def prefill_flops(lq: list[int], lk: list[int], hq: int, d: int) -> int:
    """4*Hq*D flops (QK^T and PV) per unmasked (query, key) pair."""
    pairs = sum(q * (k - q) + q * (q + 1) // 2 for q, k in zip(lq, lk))
    return 4 * hq * d * pairs
