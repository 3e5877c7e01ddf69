"""Varlen causal GQA prefill on the GPU, through the C ABI, against the fp32 CPU oracle."""
import pytest
import torch

from conftest import assert_close_to_oracle
from nano_vllm_b200 import _lib, attention as A, workloads as W
from oracle import paged_attention_ref as R

pytestmark = pytest.mark.gpu


def _check(cuda, case, what):
    dev = case.to(cuda)
    if case.k_cache.numel():
        A.store_kvcache(dev.k, dev.v, dev.k_cache, dev.v_cache, dev.slot_mapping)
        R.store_kvcache_ref(case.k, case.v, case.k_cache, case.v_cache, case.slot_mapping)
    if case.block_tables is not None:
        out = A.prefill_varlen(dev.q, dev.k_cache, dev.v_cache, dev.cu_seqlens_q, dev.cu_seqlens_k,
                               case.max_seqlen_q, case.max_seqlen_k, case.scale, block_tables=dev.block_tables)
        ref = R.prefill_ref(case.q, case.k_cache, case.v_cache, case.cu_seqlens_q, case.cu_seqlens_k, case.scale,
                            case.block_tables)
    else:
        out = A.prefill_varlen(dev.q, dev.k, dev.v, dev.cu_seqlens_q, dev.cu_seqlens_k,
                               case.max_seqlen_q, case.max_seqlen_k, case.scale)
        ref = R.prefill_ref(case.q, case.k, case.v, case.cu_seqlens_q, case.cu_seqlens_k, case.scale)
    torch.cuda.synchronize()
    assert_close_to_oracle(out, ref, what)
    if case.k_cache.numel():
        assert torch.equal(dev.k_cache.cpu().view(torch.int16), case.k_cache.view(torch.int16))
        assert torch.equal(dev.v_cache.cpu().view(torch.int16), case.v_cache.view(torch.int16))
    assert _lib.read_status() == 0


def test_cfg2(cuda):
    """The prefill configuration at full size: 64 prompts in [100,1024], every 4th shares 1-3 cached blocks."""
    case = W.cfg2_prefill()
    assert case.block_tables is not None and int(case.cu_seqlens_k[-1]) > int(case.cu_seqlens_q[-1])
    _check(cuda, case, "cfg2")


@pytest.mark.parametrize("hq,hkv,d", [(16, 8, 128), (32, 8, 128), (14, 2, 64), (4, 1, 128), (2, 2, 64),
                                      (8, 1, 128), (12, 2, 64), (16, 2, 64), (10, 2, 128), (6, 2, 128), (14, 2, 128)])
def test_packed_lengths(cuda, hq, hkv, d):
    case = W.make_prefill_case(21, 8, 1, 1, hq, hkv, d, share_every=0,
                               lengths=[1, 100, 127, 128, 129, 256, 257, 1024])
    assert case.block_tables is None
    _check(cuda, case, f"packed hq{hq} hkv{hkv} d{d}")


@pytest.mark.parametrize("d", [64, 128])
def test_prefix_cached_blocks(cuda, d):
    """Lk - Lq in {0, 256, 768}; a fully cached prompt leaves Lq == 0."""
    case = W.make_prefill_case(22, 6, 1, 1, 8, 2, d, lengths=[1024, 1024, 300, 257, 512, 512],
                               shared_blocks=[0, 3, 0, 1, 0, 2])
    lq = (case.cu_seqlens_q[1:] - case.cu_seqlens_q[:-1]).tolist()
    assert lq == [1024, 256, 300, 1, 512, 0]
    _check(cuda, case, f"prefix d{d}")


def test_warmup_shape_without_cache(cuda):
    """Engine warm-up: 4096-token sequences before the cache exists
    (nanovllm/engine/model_runner.py:96-108)."""
    case = W.make_prefill_case(23, 2, 1, 1, 16, 8, 128, lengths=[4096, 4096], with_cache=False)
    _check(cuda, case, "warmup")


def test_strided_v_view(cuda):
    hq, hkv, d, n = 16, 8, 128, 700
    g = torch.Generator().manual_seed(24)
    qkv = torch.randn(n, (hq + 2 * hkv) * d, generator=g).bfloat16()
    cu = torch.tensor([0, 300, 700], dtype=torch.int32)
    q, k, v = (t.view(n, -1, d) for t in qkv.split([hq * d, hkv * d, hkv * d], dim=-1))
    qd, kd, vd = (t.view(n, -1, d) for t in qkv.to(cuda).split([hq * d, hkv * d, hkv * d], dim=-1))
    out = A.prefill_varlen(qd, kd, vd, cu.to(cuda), cu.to(cuda), 400, 400, d ** -0.5)
    ref = R.prefill_ref(q, k, v, cu, cu, d ** -0.5)
    assert_close_to_oracle(out, ref, "strided")


@pytest.mark.parametrize("d", [64, 128])
def test_stale_cache_rows_past_the_sequence_cannot_leak(cuda, d):
    """A partly filled last block holds NaN/Inf past the sequence end; outputs stay finite."""
    case = W.make_prefill_case(25, 3, 1, 1, 8, 2, d, lengths=[300, 700, 513], shared_blocks=[0, 1, 2])
    assert case.block_tables is not None
    case.k_cache[:] = float("nan")
    case.v_cache[:] = float("inf")
    _check(cuda, case, f"stale d{d}")


@pytest.mark.parametrize("impl,d", [("mma", 64), ("mma", 128), ("tcp", 64), ("tcp", 128)])
def test_every_prefill_kernel_on_the_same_case(cuda, monkeypatch, impl, d):
    """NVLLM_PREFILL_IMPL=mma selects the warp-level cross-check kernel instead of the persistent
    tcgen05 kernel (tcp, the default); both must agree with the oracle on packed and on
    prefix-cached inputs."""
    monkeypatch.setenv("NVLLM_PREFILL_IMPL", impl)
    case = W.make_prefill_case(26, 7, 1, 1, 8, 2, d, lengths=[1, 130, 1024, 1024, 513, 700, 64],
                               shared_blocks=[0, 0, 0, 3, 0, 2, 0])
    _check(cuda, case, f"{impl} d{d} prefix")
    case = W.make_prefill_case(27, 5, 1, 1, 8, 8, d, share_every=0, lengths=[257, 2, 900, 128, 64])
    _check(cuda, case, f"{impl} d{d} packed")


def test_many_sequences_through_the_persistent_kernel(cuda):
    """More work items than resident blocks, and more sequences than one warp scans at once."""
    case = W.make_prefill_case(28, 150, 1, 300, 4, 2, 128, share_every=0)
    _check(cuda, case, "150 sequences")


@pytest.mark.parametrize("cap", [1, 2, 3, 4, 8])
@pytest.mark.parametrize("d", [64, 128])
def test_head_packing_of_the_persistent_kernel(cuda, monkeypatch, cap, d):
    """The persistent kernel packs up to 8 query heads of one KV head into the 128 rows of a tile
    (16 to 128 tokens per tile; the number of heads is the largest divisor of the group size
    within the cap, so 3, 5, 6 or 7 heads leave a few rows unused); NVLLM_PREFILL_PACK caps the
    number.  Every packing must agree with the oracle on ragged packed input and on
    prefix-cached input."""
    monkeypatch.setenv("NVLLM_PREFILL_IMPL", "tcp")
    monkeypatch.setenv("NVLLM_PREFILL_PACK", str(cap))
    case = W.make_prefill_case(28, 9, 1, 1, 16, 2, d, share_every=0,
                               lengths=[1, 15, 16, 17, 33, 130, 511, 1024, 700])
    _check(cuda, case, f"packed cap{cap} d{d}")
    case = W.make_prefill_case(29, 5, 1, 1, 16, 2, d, lengths=[1024, 1024, 300, 257, 600],
                               shared_blocks=[0, 3, 0, 1, 0])
    _check(cuda, case, f"paged cap{cap} d{d}")
