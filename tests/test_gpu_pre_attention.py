"""Fused q/k RMSNorm + rotary embedding + KV-cache store on the GPU against the CPU
restatement of the reference's separate ops."""
import sys
from pathlib import Path

import pytest
import torch

sys.path.insert(0, str(Path(__file__).resolve().parent / "golden"))
import cases as C  # noqa: E402

from nano_vllm_b200 import _lib, attention as A
from oracle import paged_attention_ref as R

pytestmark = pytest.mark.gpu


def _bf16_ulp_close(got, ref, what):
    """Same roundings as the reference, different summation order inside the norm: in rare
    elements the normalised value lands on the neighbouring bf16, and the rotation carries that
    one-ulp step of an input (x1, x2) into both outputs.  So the bound is one bf16 ulp of the
    rotated pair's magnitude (a rotation keeps |(x1, x2)|), never more, and almost every element
    must be bit-identical."""
    got, ref = got.float().cpu(), ref.float()
    half = ref.shape[-1] // 2
    mag = (ref[..., :half] ** 2 + ref[..., half:] ** 2).sqrt()
    tol = torch.cat([mag, mag], dim=-1) * 2.0 ** -7 + 1e-6
    bad = (got - ref).abs() > tol
    assert not bad.any(), f"{what}: {int(bad.sum())} elements off by more than one bf16 ulp of their pair"
    exact = (got == ref).float().mean().item()
    assert exact > 0.99, f"{what}: only {exact:.4f} of the elements are bit-identical"


@pytest.mark.parametrize("hq,hkv,d,norm", [(16, 8, 128, True), (4, 1, 128, True), (14, 2, 64, False), (2, 2, 64, True)])
def test_fused_pre_attention_matches_the_separate_reference_ops(cuda, hq, hkv, d, norm):
    g = torch.Generator().manual_seed(81 + hq + d)
    n, max_pos, eps = 333, 4096, 1e-6
    qkv = (torch.randn(n, (hq + 2 * hkv) * d, generator=g) * 3).bfloat16()
    positions = torch.randint(0, max_pos, (n,), generator=g)
    qw = (1 + 0.1 * torch.randn(d, generator=g)).bfloat16() if norm else None
    kw = (1 + 0.1 * torch.randn(d, generator=g)).bfloat16() if norm else None
    cache = R.rotary_cache_ref(d, max_pos, 1e6)
    k_cache = torch.randn(3, 256, hkv, d, generator=g).bfloat16()
    v_cache = torch.randn(3, 256, hkv, d, generator=g).bfloat16()
    slots = torch.randperm(3 * 256, generator=g)[:n].to(torch.int32)
    slots[::29] = -1

    q_ref, k_ref, v_ref = R.qk_norm_rope_ref(qkv, positions, qw, kw, cache, eps, hq, hkv, d)
    kc_ref, vc_ref = k_cache.clone(), v_cache.clone()
    R.store_kvcache_ref(k_ref, v_ref, kc_ref, vc_ref, slots)

    qkv_d, kc, vc = qkv.to(cuda), k_cache.to(cuda), v_cache.to(cuda)
    A.qk_norm_rope_store(qkv_d, positions.to(cuda), qw.to(cuda) if norm else None, kw.to(cuda) if norm else None,
                         cache.to(cuda), eps, slots.to(cuda), kc, vc, hq, hkv, d)
    torch.cuda.synchronize()
    q_d, k_d, v_d = qkv_d.cpu().split([hq * d, hkv * d, hkv * d], dim=-1)
    _bf16_ulp_close(q_d.reshape(n, hq, d), q_ref, "q")
    _bf16_ulp_close(k_d.reshape(n, hkv, d), k_ref, "k")
    assert torch.equal(v_d.reshape(n, hkv, d).view(torch.int16), v_ref.view(torch.int16)), "v must be untouched"
    # the cache holds exactly what the kernel left in the qkv buffer (the copy is bit-exact),
    # and untouched slots are untouched
    kc_expect, vc_expect = k_cache.clone(), v_cache.clone()
    R.store_kvcache_ref(k_d.reshape(n, hkv, d).contiguous(), v_d.reshape(n, hkv, d).contiguous(), kc_expect, vc_expect, slots)
    assert torch.equal(kc.cpu().view(torch.int16), kc_expect.view(torch.int16))
    assert torch.equal(vc.cpu().view(torch.int16), vc_expect.view(torch.int16))
    _bf16_ulp_close(kc.cpu(), kc_ref, "k_cache")
    assert _lib.read_status() == 0


def test_fused_pre_attention_without_a_cache_is_rotation_only(cuda):
    """Engine warm-up: no cache yet, empty slot_mapping (nanovllm/engine/model_runner.py:96-108)."""
    g = torch.Generator().manual_seed(90)
    hq, hkv, d, n = 16, 8, 128, 64
    qkv = torch.randn(n, (hq + 2 * hkv) * d, generator=g).bfloat16()
    positions = torch.arange(n)
    w = torch.ones(d).bfloat16()
    cache = R.rotary_cache_ref(d, 256, 1e6)
    q_ref, k_ref, _ = R.qk_norm_rope_ref(qkv, positions, w, w, cache, 1e-6, hq, hkv, d)
    qkv_d = qkv.to(cuda)
    empty = torch.zeros(0, dtype=torch.bfloat16, device=cuda)
    A.qk_norm_rope_store(qkv_d, positions.to(cuda), w.to(cuda), w.to(cuda), cache.to(cuda), 1e-6,
                         torch.zeros(0, dtype=torch.int32, device=cuda), empty, empty, hq, hkv, d)
    q_d, k_d, _ = qkv_d.cpu().split([hq * d, hkv * d, hkv * d], dim=-1)
    _bf16_ulp_close(q_d.reshape(n, hq, d), q_ref, "q")
    _bf16_ulp_close(k_d.reshape(n, hkv, d), k_ref, "k")


@pytest.mark.parametrize("name", ["qwen2", "qwen3", "qwen3_8b_shard"])
def test_recorded_reference_modules(cuda, name):
    """Inputs for which the output of nano-vllm's own RMSNorm and RotaryEmbedding modules was
    recorded (tests/golden/make_pre_attention_golden.py)."""
    c = C.pre_attention_cases()[name]
    hq, hkv, d, n = c["hq"], c["hkv"], c["d"], c["qkv"].shape[0]
    cache = R.rotary_cache_ref(d, c["max_pos"], c["base"]).to(cuda)
    qkv = c["qkv"].to(cuda)
    empty = torch.zeros(0, dtype=torch.bfloat16, device=cuda)
    A.qk_norm_rope_store(qkv, c["positions"].to(cuda), c["q_weight"].to(cuda) if c["q_weight"] is not None else None,
                         c["k_weight"].to(cuda) if c["k_weight"] is not None else None, cache, 1e-6,
                         torch.zeros(0, dtype=torch.int32, device=cuda), empty, empty, hq, hkv, d)
    q_d, k_d, v_d = qkv.cpu().split([hq * d, hkv * d, hkv * d], dim=-1)
    _bf16_ulp_close(q_d.reshape(n, hq, d), c["q"], "q")
    _bf16_ulp_close(k_d.reshape(n, hkv, d), c["k"], "k")
    assert torch.equal(v_d, c["qkv"][:, (hq + hkv) * d:])
