"""store_kvcache on the GPU, through the C ABI, bit-exact against the CPU oracle."""
import pytest
import torch

from nano_vllm_b200 import _lib, attention as A, workloads as W
from oracle import paged_attention_ref as R

pytestmark = pytest.mark.gpu


def _run_store(cuda, key, value, k_cache, v_cache, slots):
    kc, vc = k_cache.to(cuda), v_cache.to(cuda)
    A.store_kvcache(key.to(cuda), value.to(cuda), kc, vc, slots.to(cuda))
    torch.cuda.synchronize()
    return kc.cpu(), vc.cpu()


@pytest.mark.parametrize("hkv,d", [(8, 128), (2, 64), (1, 128), (1, 64)])
@pytest.mark.parametrize("n", [1, 7, 256, 1000])
def test_store_matches_oracle(cuda, hkv, d, n):
    g = torch.Generator().manual_seed(n * 131 + hkv)
    num_blocks = (n + 255) // 256 + 3
    key = torch.randn(n, hkv, d, generator=g).bfloat16()
    value = torch.randn(n, hkv, d, generator=g).bfloat16()
    k_cache = torch.randn(num_blocks, 256, hkv, d, generator=g).bfloat16()
    v_cache = torch.randn(num_blocks, 256, hkv, d, generator=g).bfloat16()
    slots = torch.randperm(num_blocks * 256, generator=g)[:n].to(torch.int32)
    kc, vc = _run_store(cuda, key, value, k_cache, v_cache, slots)
    R.store_kvcache_ref(key, value, k_cache, v_cache, slots)
    assert torch.equal(kc.view(torch.int16), k_cache.view(torch.int16))  # untouched slots included
    assert torch.equal(vc.view(torch.int16), v_cache.view(torch.int16))
    assert _lib.read_status() == 0


def test_store_strided_value_and_negative_slot(cuda):
    """value is a strided view of a fused qkv activation (nanovllm/models/qwen3.py:89);
    slot -1 rows are skipped."""
    g = torch.Generator().manual_seed(5)
    n, hq, hkv, d = 300, 16, 8, 128
    qkv = torch.randn(n, (hq + 2 * hkv) * d, generator=g).bfloat16()
    q, k, v = qkv.split([hq * d, hkv * d, hkv * d], dim=-1)
    k, v = k.view(n, hkv, d), v.view(n, hkv, d)
    k_cache = torch.zeros(4, 256, hkv, d).bfloat16()
    v_cache = torch.zeros(4, 256, hkv, d).bfloat16()
    slots = torch.randperm(4 * 256, generator=g)[:n].to(torch.int32)
    slots[::17] = -1
    qkv_d = qkv.to(cuda)
    _, kd, vd = qkv_d.split([hq * d, hkv * d, hkv * d], dim=-1)
    kc, vc = k_cache.to(cuda), v_cache.to(cuda)
    A.store_kvcache(kd.view(n, hkv, d), vd.view(n, hkv, d), kc, vc, slots.to(cuda))
    R.store_kvcache_ref(k, v, k_cache, v_cache, slots)
    assert torch.equal(kc.cpu().view(torch.int16), k_cache.view(torch.int16))
    assert torch.equal(vc.cpu().view(torch.int16), v_cache.view(torch.int16))


def test_store_out_of_range_slot_is_skipped_and_flagged(cuda):
    n, hkv, d = 4, 2, 64
    key = torch.ones(n, hkv, d).bfloat16().to(cuda)
    kc = torch.zeros(1, 256, hkv, d).bfloat16().to(cuda)
    vc = torch.zeros_like(kc)
    slots = torch.tensor([0, 256, 3, 100000], dtype=torch.int32).to(cuda)
    _lib.read_status()
    A.store_kvcache(key, key, kc, vc, slots)
    assert _lib.read_status() & 1
    flat = kc.view(256, -1).float().sum(1).cpu()
    assert flat[0] > 0 and flat[3] > 0 and (flat > 0).sum() == 2


def test_store_duplicate_slots(cuda):
    """Graph padding rows all target slot 0 with identical data
    (nanovllm/engine/model_runner.py:271-276): the slot must hold exactly that row.  When the
    duplicate writers differ (never produced by the runner) every 16-byte piece must still
    come whole from one of them."""
    n, hkv, d = 64, 8, 128
    same = torch.full((n, hkv, d), 3.0).bfloat16().to(cuda)
    kc = torch.full((1, 256, hkv, d), -1.0).bfloat16().to(cuda)
    vc = torch.full_like(kc, -1.0)
    zeros = torch.zeros(n, dtype=torch.int32, device=cuda)
    A.store_kvcache(same, same, kc, vc, zeros)
    assert (kc.view(256, -1)[0] == 3.0).all() and (vc.view(256, -1)[0] == 3.0).all()
    assert (kc.view(256, -1)[1:] == -1.0).all()
    key = torch.arange(n).view(n, 1, 1).expand(n, hkv, d).bfloat16().contiguous().to(cuda)
    A.store_kvcache(key, key, kc, vc, zeros)
    pieces = kc.view(256, -1)[0].float().cpu().view(-1, 8)
    assert (pieces.min(1).values == pieces.max(1).values).all()
    assert ((pieces[:, 0] >= 0) & (pieces[:, 0] < n)).all()


def test_store_empty_and_cfg2_full_size(cuda):
    case = W.cfg2_prefill()
    kc, vc = _run_store(cuda, case.k, case.v, case.k_cache, case.v_cache, case.slot_mapping)
    R.store_kvcache_ref(case.k, case.v, case.k_cache, case.v_cache, case.slot_mapping)
    assert torch.equal(kc.view(torch.int16), case.k_cache.view(torch.int16))
    assert torch.equal(vc.view(torch.int16), case.v_cache.view(torch.int16))
    empty = torch.zeros(0, 8, 128).bfloat16().to(cuda)
    A.store_kvcache(empty, empty, kc.to(cuda), vc.to(cuda), torch.zeros(0, dtype=torch.int32, device=cuda))
