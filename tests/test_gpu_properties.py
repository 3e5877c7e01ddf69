"""Property tests over random lengths, prefix hits and scattered block tables, and canary
checks that no kernel writes outside the rows it owns (no memory checker is available where these
tests run, so out-of-bounds writes are looked for with sentinels around every output)."""
import pytest
import torch
from hypothesis import given, settings, strategies as st, HealthCheck

from conftest import assert_close_to_oracle
from nano_vllm_b200 import _lib, attention as A, workloads as W
from oracle import paged_attention_ref as R

pytestmark = pytest.mark.gpu

GEOMS = [(16, 8, 128), (32, 8, 128), (14, 2, 64), (4, 4, 128), (8, 1, 64)]
COMMON = dict(deadline=None, derandomize=True, suppress_health_check=[HealthCheck.function_scoped_fixture, HealthCheck.too_slow])


@settings(max_examples=25, **COMMON)
@given(seed=st.integers(0, 10 ** 6), geom=st.sampled_from(GEOMS),
       lens=st.lists(st.one_of(st.integers(0, 40), st.integers(200, 300), st.integers(500, 2100)), min_size=1, max_size=9),
       extra_width=st.integers(0, 6))
def test_decode_matches_oracle_for_any_lengths(cuda, seed, geom, lens, extra_width):
    hq, hkv, d = geom
    width = max((max(lens) + 255) // 256, 1) + extra_width
    case = W.make_decode_case(seed, len(lens), 1, 1, hq, hkv, d, context_lens=lens, table_width=width)
    case.block_tables[case.context_lens == 0] = 0  # graph-padding rows look like this
    dev = case.to(cuda)
    out = A.decode_paged(dev.q, dev.k_cache, dev.v_cache, dev.context_lens, dev.block_tables, case.scale)
    ref = R.decode_ref(case.q, case.k_cache, case.v_cache, case.context_lens, case.block_tables, case.scale)
    assert_close_to_oracle(out, ref, f"decode {geom} {lens} width {width}")
    assert _lib.read_status() == 0


@settings(max_examples=20, **COMMON)
@given(seed=st.integers(0, 10 ** 6), geom=st.sampled_from(GEOMS), data=st.data())
def test_prefill_matches_oracle_for_any_lengths_and_prefix_hits(cuda, seed, geom, data):
    hq, hkv, d = geom
    n = data.draw(st.integers(1, 6))
    lens = [data.draw(st.one_of(st.integers(1, 130), st.integers(250, 260), st.integers(300, 1100))) for _ in range(n)]
    shared = [0] * n
    for i in range(1, n):
        most = min(lens[i - 1] // 256, lens[i] // 256)  # whole blocks of the predecessor; Lq == 0 is allowed
        if most and shared[i - 1] == 0:
            shared[i] = data.draw(st.integers(0, most))
    case = W.make_prefill_case(seed, n, 1, 1, hq, hkv, d, lengths=lens, shared_blocks=shared)
    dev = case.to(cuda)
    A.store_kvcache(dev.k, dev.v, dev.k_cache, dev.v_cache, dev.slot_mapping)
    R.store_kvcache_ref(case.k, case.v, case.k_cache, case.v_cache, case.slot_mapping)
    if case.block_tables is not None:
        out = A.prefill_varlen(dev.q, dev.k_cache, dev.v_cache, dev.cu_seqlens_q, dev.cu_seqlens_k, case.max_seqlen_q,
                               case.max_seqlen_k, case.scale, block_tables=dev.block_tables)
        ref = R.prefill_ref(case.q, case.k_cache, case.v_cache, case.cu_seqlens_q, case.cu_seqlens_k, case.scale,
                            case.block_tables)
    else:
        out = A.prefill_varlen(dev.q, dev.k, dev.v, dev.cu_seqlens_q, dev.cu_seqlens_k, case.max_seqlen_q,
                               case.max_seqlen_k, case.scale)
        ref = R.prefill_ref(case.q, case.k, case.v, case.cu_seqlens_q, case.cu_seqlens_k, case.scale)
    if case.q.shape[0]:
        assert_close_to_oracle(out, ref, f"prefill {geom} {lens} shared {shared}")
    assert torch.equal(dev.k_cache.cpu().view(torch.int16), case.k_cache.view(torch.int16))
    assert _lib.read_status() == 0


def _guarded(shape, device, fill=-7.0):
    """A tensor of `shape` carved out of a larger buffer whose surroundings hold a sentinel."""
    n = 1
    for s in shape:
        n *= s
    pad = 4096
    buf = torch.full((n + 2 * pad,), fill, dtype=torch.bfloat16, device=device)
    return buf, buf[pad:pad + n].view(shape), pad


def _guards_intact(buf, pad, fill=-7.0):
    return bool((buf[:pad] == fill).all() and (buf[-pad:] == fill).all())


@pytest.mark.parametrize("hq,hkv,d", GEOMS)
def test_no_kernel_writes_outside_its_output(cuda, hq, hkv, d):
    # decode: rows of `out` only
    dc = W.make_decode_case(95, 5, 1, 1, hq, hkv, d, context_lens=[1, 300, 0, 1025, 77], table_width=9)
    dc.block_tables[2] = 0
    dd = dc.to(cuda)
    buf, out, pad = _guarded((5, hq, d), cuda)
    A.decode_paged(dd.q, dd.k_cache, dd.v_cache, dd.context_lens, dd.block_tables, dc.scale, out=out)
    torch.cuda.synchronize()
    assert _guards_intact(buf, pad), "decode wrote outside out"
    # prefill: rows past each sequence's end (the tail of a 128-row tile) must not be written;
    # here the last sequence ends 3 rows into a tile and the guard follows immediately
    pc = W.make_prefill_case(96, 3, 1, 1, hq, hkv, d, share_every=0, lengths=[130, 1, 259])
    pd = pc.to(cuda)
    n = pc.q.shape[0]
    buf, out, pad = _guarded((n, hq, d), cuda)
    A.prefill_varlen(pd.q, pd.k, pd.v, pd.cu_seqlens_q, pd.cu_seqlens_k, pc.max_seqlen_q, pc.max_seqlen_k, pc.scale, out=out)
    torch.cuda.synchronize()
    assert _guards_intact(buf, pad), "prefill wrote outside out"
    ref = R.prefill_ref(pc.q, pc.k, pc.v, pc.cu_seqlens_q, pc.cu_seqlens_k, pc.scale)
    assert_close_to_oracle(out, ref, "guarded prefill")
    # store: only the addressed cache rows change
    cbuf, kc, cpad = _guarded((2, 256, hkv, d), cuda)
    vbuf, vc, _ = _guarded((2, 256, hkv, d), cuda)
    kc.zero_()
    vc.zero_()
    slots = torch.tensor([0, 511, 256, -1, 255], dtype=torch.int32, device=cuda)
    rows = torch.ones(5, hkv, d, dtype=torch.bfloat16, device=cuda)
    A.store_kvcache(rows, rows, kc, vc, slots)
    torch.cuda.synchronize()
    assert _guards_intact(cbuf, cpad) and _guards_intact(vbuf, cpad), "store wrote outside the cache"
    assert int((kc.view(512, -1).float().sum(1) > 0).sum()) == 4
