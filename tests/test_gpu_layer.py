"""Attention.forward (the reference-facing layer) on the GPU against the oracle's
restatement of the same control flow."""
import pytest
import torch

from conftest import assert_close_to_oracle
from nano_vllm_b200 import attention as A, context as C, workloads as W
from oracle import paged_attention_ref as R

pytestmark = pytest.mark.gpu


def test_prefill_then_decode_through_the_layer(cuda):
    hq, hkv, d = 16, 8, 128
    case = W.make_prefill_case(31, 8, 100, 700, hq, hkv, d)
    dev = case.to(cuda)
    layer = A.Attention(hq, d, case.scale, hkv)
    assert layer.k_cache.numel() == 0
    layer.k_cache, layer.v_cache = dev.k_cache, dev.v_cache
    C.set_context(True, dev.cu_seqlens_q, dev.cu_seqlens_k, case.max_seqlen_q, case.max_seqlen_k,
                  dev.slot_mapping, None, dev.block_tables)
    n = case.q.shape[0]
    o = layer(dev.q.view(n, -1), dev.k.view(n, -1), dev.v.view(n, -1))
    C.set_context(True, case.cu_seqlens_q, case.cu_seqlens_k, case.max_seqlen_q, case.max_seqlen_k,
                  case.slot_mapping, None, case.block_tables)
    ref = R.attention_forward_ref(case.q, case.k, case.v, case.k_cache, case.v_cache, C.get_context(), case.scale)
    assert o.shape == (n, hq * d)
    assert_close_to_oracle(o.view(n, hq, d), ref, "layer prefill")

    # one decode step on top of the prefilled cache
    B = case.cu_seqlens_k.numel() - 1
    lens = (case.cu_seqlens_k[1:] - case.cu_seqlens_k[:-1]) + 1
    g = torch.Generator().manual_seed(32)
    q1 = torch.randn(B, hq, d, generator=g).bfloat16()
    k1 = torch.randn(B, hkv, d, generator=g).bfloat16()
    v1 = torch.randn(B, hkv, d, generator=g).bfloat16()
    bt = case.block_tables
    slots = torch.zeros(B, dtype=torch.int32)
    for b in range(B):
        pos = int(lens[b]) - 1
        if pos % 256 == 0:  # needs a fresh block: take a spare one
            free = (set(range(case.k_cache.shape[0])) - set(bt[bt >= 0].tolist())).pop()
            if pos // 256 >= bt.shape[1]:
                bt = torch.cat([bt, torch.full((B, 1), -1, dtype=torch.int32)], dim=1)
            bt[b, pos // 256] = free
        slots[b] = int(bt[b, pos // 256]) * 256 + pos % 256
    C.set_context(False, slot_mapping=slots.to(cuda), context_lens=lens.to(torch.int32).to(cuda),
                  block_tables=bt.to(cuda))
    o1 = layer(q1.to(cuda).view(B, -1), k1.to(cuda).view(B, -1), v1.to(cuda).view(B, -1))
    C.set_context(False, slot_mapping=slots, context_lens=lens.to(torch.int32), block_tables=bt)
    ref1 = R.attention_forward_ref(q1, k1, v1, case.k_cache, case.v_cache, C.get_context(), case.scale)
    C.reset_context()
    assert_close_to_oracle(o1.view(B, hq, d), ref1, "layer decode")
    assert torch.equal(dev.k_cache.cpu().view(torch.int16), case.k_cache.view(torch.int16))
