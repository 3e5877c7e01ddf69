"""CUDA kernels, through the C ABI, against outputs recorded from the reference
implementation (tests/golden/README.md)."""
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

sys.path.insert(0, str(Path(__file__).resolve().parent / "golden"))
import cases as C  # noqa: E402

from conftest import assert_close_to_oracle
from nano_vllm_b200 import attention as A, context as CTX

pytestmark = pytest.mark.gpu


def _load(name):
    z = np.load(C.GOLDEN_DIR / f"{name}.npz")
    return {k: z[k] for k in z.files}


def _gold_out(gold):
    return torch.from_numpy(gold["out"].copy()).view(torch.bfloat16).float()


@pytest.mark.parametrize("name", sorted(C.store_cases()))
def test_store_bit_exact_with_reference(cuda, name):
    key, value, k_cache, v_cache, slots = C.store_cases()[name]
    gold = _load(name)
    n, hkv, d = key.shape
    kv = torch.cat([key.reshape(n, -1), value.reshape(n, -1)], dim=1).to(cuda)
    kd, vd = (t.view(n, hkv, d) for t in kv.split(hkv * d, dim=-1))
    kc, vc = k_cache.to(cuda), v_cache.to(cuda)
    A.store_kvcache(kd, vd, kc, vc, slots.to(cuda))
    assert C.sha(kc.cpu()) == str(gold["k_cache_sha"]) and C.sha(vc.cpu()) == str(gold["v_cache_sha"])


@pytest.mark.parametrize("name", sorted(C.decode_cases()))
def test_decode_layer_matches_reference(cuda, name):
    case = C.decode_cases()[name]
    gold = _load(name)
    d = case.to(cuda)
    B, Hq, Hkv, D = case.geometry
    layer = A.Attention(Hq, D, case.scale, Hkv)
    layer.k_cache, layer.v_cache = d.k_cache, d.v_cache
    CTX.set_context(False, slot_mapping=d.slot_mapping, context_lens=d.context_lens, block_tables=d.block_tables)
    o = layer(d.q.view(B, -1), d.k_new.view(B, -1), d.v_new.view(B, -1))
    CTX.reset_context()
    assert C.sha(d.k_cache.cpu()) == str(gold["k_cache_sha"]) and C.sha(d.v_cache.cpu()) == str(gold["v_cache_sha"])
    assert_close_to_oracle(o.view(B, Hq, D), _gold_out(gold), name)


@pytest.mark.parametrize("name", sorted(C.prefill_cases()))
def test_prefill_layer_matches_reference(cuda, name):
    case = C.prefill_cases()[name]
    gold = _load(name)
    d = case.to(cuda)
    N, Hq, D = case.q.shape
    Hkv = case.k.shape[1]
    layer = A.Attention(Hq, D, case.scale, Hkv)
    layer.k_cache, layer.v_cache = d.k_cache, d.v_cache
    CTX.set_context(True, d.cu_seqlens_q, d.cu_seqlens_k, case.max_seqlen_q, case.max_seqlen_k, d.slot_mapping,
                    None, d.block_tables)
    o = layer(d.q.view(N, -1), d.k.view(N, -1), d.v.view(N, -1))
    CTX.reset_context()
    assert C.sha(d.k_cache.cpu()) == str(gold["k_cache_sha"]) and C.sha(d.v_cache.cpu()) == str(gold["v_cache_sha"])
    assert_close_to_oracle(o.view(N, Hq, D), _gold_out(gold), name)


@pytest.mark.parametrize("name", sorted(C.prefill_cases()) + sorted(C.decode_cases()))
def test_no_less_accurate_than_the_reference_kernels(cuda, name):
    """Against the fp32 oracle, the new kernels' error must not exceed that of the reference's
    own kernels (flash-attn, recorded in the golden files) by more than rounding noise."""
    from oracle import paged_attention_ref as R
    gold = _load(name)
    if name in C.decode_cases():
        case = C.decode_cases()[name]
        d = case.to(cuda)
        A.store_kvcache(d.k_new, d.v_new, d.k_cache, d.v_cache, d.slot_mapping)
        R.store_kvcache_ref(case.k_new, case.v_new, case.k_cache, case.v_cache, case.slot_mapping)
        ours = A.decode_paged(d.q, d.k_cache, d.v_cache, d.context_lens, d.block_tables, case.scale)
        ref = R.decode_ref(case.q, case.k_cache, case.v_cache, case.context_lens, case.block_tables, case.scale)
    else:
        case = C.prefill_cases()[name]
        d = case.to(cuda)
        A.store_kvcache(d.k, d.v, d.k_cache, d.v_cache, d.slot_mapping)
        R.store_kvcache_ref(case.k, case.v, case.k_cache, case.v_cache, case.slot_mapping)
        if case.block_tables is not None:
            ours = A.prefill_varlen(d.q, d.k_cache, d.v_cache, d.cu_seqlens_q, d.cu_seqlens_k, case.max_seqlen_q,
                                    case.max_seqlen_k, case.scale, block_tables=d.block_tables)
            ref = R.prefill_ref(case.q, case.k_cache, case.v_cache, case.cu_seqlens_q, case.cu_seqlens_k, case.scale,
                                case.block_tables)
        else:
            ours = A.prefill_varlen(d.q, d.k, d.v, d.cu_seqlens_q, d.cu_seqlens_k, case.max_seqlen_q,
                                    case.max_seqlen_k, case.scale)
            ref = R.prefill_ref(case.q, case.k, case.v, case.cu_seqlens_q, case.cu_seqlens_k, case.scale)
    ours_err = (ours.float().cpu() - ref).abs()
    gold_err = (_gold_out(gold) - ref).abs()
    print(f"{name}: mean-abs ours {ours_err.mean():.3e} reference {gold_err.mean():.3e}; "
          f"max-abs ours {ours_err.max():.3e} reference {gold_err.max():.3e}")
    assert ours_err.mean() <= 1.25 * gold_err.mean() + 1e-5
    assert ours_err.max() <= 2.0 * gold_err.max() + 1e-3
