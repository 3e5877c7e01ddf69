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
