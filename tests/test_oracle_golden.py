"""Pins the CPU oracle to outputs recorded from the reference implementation itself
(tests/golden/README.md).  Runs without a GPU."""
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

sys.path.insert(0, str(Path(__file__).resolve().parent / "golden"))
import cases as C  # noqa: E402

from conftest import assert_close_to_oracle
from oracle import paged_attention_ref as R


def _load(name):
    z = np.load(C.GOLDEN_DIR / f"{name}.npz")
    return {k: z[k] for k in z.files}


def _bf16(a):
    return torch.from_numpy(a.copy()).view(torch.bfloat16)


@pytest.mark.parametrize("name", sorted(C.store_cases()))
def test_store_digest_matches_reference(name):
    key, value, k_cache, v_cache, slots = C.store_cases()[name]
    gold = _load(name)
    assert str(gold["inputs"]) == C.input_fingerprint(key, value, k_cache, v_cache, slots), "seeded inputs drifted"
    R.store_kvcache_ref(key, value, k_cache, v_cache, slots)
    assert C.sha(k_cache) == str(gold["k_cache_sha"])
    assert C.sha(v_cache) == str(gold["v_cache_sha"])


@pytest.mark.parametrize("name", sorted(C.decode_cases()))
def test_decode_oracle_matches_reference(name):
    case = C.decode_cases()[name]
    gold = _load(name)
    assert str(gold["inputs"]) == C.input_fingerprint(case.q, case.k_new, case.v_new, case.k_cache, case.v_cache,
                                                      case.context_lens, case.block_tables, case.slot_mapping)
    R.store_kvcache_ref(case.k_new, case.v_new, case.k_cache, case.v_cache, case.slot_mapping)
    assert C.sha(case.k_cache) == str(gold["k_cache_sha"]) and C.sha(case.v_cache) == str(gold["v_cache_sha"])
    ref = R.decode_ref(case.q, case.k_cache, case.v_cache, case.context_lens, case.block_tables, case.scale)
    assert_close_to_oracle(_bf16(gold["out"]), ref, name)


@pytest.mark.parametrize("name", sorted(C.prefill_cases()))
def test_prefill_oracle_matches_reference(name):
    case = C.prefill_cases()[name]
    gold = _load(name)
    assert str(gold["inputs"]) == C.input_fingerprint(case.q, case.k, case.v, case.cu_seqlens_q, case.cu_seqlens_k,
                                                      case.slot_mapping, case.block_tables)
    R.store_kvcache_ref(case.k, case.v, case.k_cache, case.v_cache, case.slot_mapping)
    assert C.sha(case.k_cache) == str(gold["k_cache_sha"]) and C.sha(case.v_cache) == str(gold["v_cache_sha"])
    if case.block_tables is not None:
        ref = R.prefill_ref(case.q, case.k_cache, case.v_cache, case.cu_seqlens_q, case.cu_seqlens_k, case.scale,
                            case.block_tables)
    else:
        ref = R.prefill_ref(case.q, case.k, case.v, case.cu_seqlens_q, case.cu_seqlens_k, case.scale)
    assert_close_to_oracle(_bf16(gold["out"]), ref, name)


@pytest.mark.parametrize("name", ["ragged_vocab", "small", "wide"])
def test_sampler_oracle_matches_reference(name):
    """Tokens that nano-vllm's own Sampler returned on the CPU for a recorded exponential draw."""
    logits, temperatures, noise, tokens = C.sampler_cases()[name]
    assert torch.equal(R.sampler_ref(logits, temperatures, noise), tokens)
    greedy = temperatures == 0
    assert greedy.any() and torch.equal(tokens[greedy], logits.float().argmax(-1)[greedy])


@pytest.mark.parametrize("name", ["few", "graph_batch", "one", "ragged"])
def test_decode_inputs_oracle_matches_reference(name):
    """The restated buffer contents against what nano-vllm's own prepare_decode returned."""
    seqs, rec = C.decode_input_cases()[name]
    n, widest = len(seqs), rec["block_tables"].shape[1]
    ref = R.decode_inputs_ref(seqs, n + 3, widest + 2)   # a graph batch and a table wider than the step
    for k in ("input_ids", "positions", "slot_mapping", "context_lens"):
        assert ref[k].dtype == rec[k].dtype and np.array_equal(ref[k][:n], rec[k]), k
        assert not ref[k][n:].any()
    assert np.array_equal(ref["block_tables"][:n, :widest], rec["block_tables"])
    assert not ref["block_tables"][:, widest:].any() and not ref["block_tables"][n:].any()


@pytest.mark.parametrize("name", ["qwen2", "qwen3", "qwen3_8b_shard"])
def test_pre_attention_oracle_matches_reference(name):
    """q/k RMSNorm + rotary embedding: the restatement against nano-vllm's own modules, bit for bit."""
    c = C.pre_attention_cases()[name]
    cache = R.rotary_cache_ref(c["d"], c["max_pos"], c["base"])
    rows = torch.tensor([0, 1, c["max_pos"] // 2, c["max_pos"] - 1])
    assert torch.equal(cache[rows], c["cache_rows"])
    q, k, v = R.qk_norm_rope_ref(c["qkv"], c["positions"], c["q_weight"], c["k_weight"], cache, 1e-6, c["hq"], c["hkv"], c["d"])
    assert torch.equal(q.view(torch.int16), c["q"].view(torch.int16))
    assert torch.equal(k.view(torch.int16), c["k"].view(torch.int16))
    assert torch.equal(v.reshape(v.shape[0], -1), c["qkv"][:, (c["hq"] + c["hkv"]) * c["d"]:])


def _lm_head_case(z, name):
    ranks, vocab, hidden, rows = (int(v) for v in z[f"{name}.shape"])
    seed, noise_seed = (int(v) for v in z[f"{name}.seeds"])
    g = torch.Generator().manual_seed(seed)
    weight = torch.randn(vocab, hidden, generator=g).to(torch.bfloat16)
    x = torch.randn(rows, hidden, generator=g).to(torch.bfloat16)
    lens = z[f"{name}.lens"].tolist()
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32) if lens else None
    temps = torch.from_numpy(z[f"{name}.temperatures"])
    torch.manual_seed(noise_seed)
    noise = torch.empty(temps.numel(), vocab, dtype=torch.float32).exponential_(1)
    return ranks, weight, x, cu, temps, noise


def test_lm_head_and_sampler_oracle_reproduces_the_reference_under_emulated_ranks():
    """oracle.lm_head_sample_ref against the tokens of nano-vllm's own ParallelLMHead + Sampler run
    with 1, 2, 4 and 8 emulated ranks (tests/golden/make_lm_head_golden.py), prefill and decode."""
    z = np.load(C.GOLDEN_DIR / "lm_head.npz")
    names = sorted({k.split(".")[0] for k in z.files})
    assert len(names) >= 6
    for name in names:
        ranks, weight, x, cu, temps, noise = _lm_head_case(z, name)
        shards = list(weight.chunk(ranks, 0))
        tokens, logits = R.lm_head_sample_ref(x, shards, cu, temps, noise)
        assert tokens.tolist() == z[f"{name}.tokens"].tolist(), name
        if f"{name}.logits" in z.files:
            assert torch.equal(logits.view(torch.int16), torch.from_numpy(z[f"{name}.logits"])), name
