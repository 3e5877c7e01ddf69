"""Paged GQA decode on the GPU, through the C ABI, against the fp32 CPU oracle."""
import pytest
import torch

from conftest import assert_close_to_oracle
from nano_vllm_b200 import _lib, attention as A, workloads as W
from oracle import paged_attention_ref as R

pytestmark = pytest.mark.gpu


def _check(cuda, case, what, store_first=True):
    dev = case.to(cuda)
    if store_first:
        A.store_kvcache(dev.k_new, dev.v_new, dev.k_cache, dev.v_cache, dev.slot_mapping)
        R.store_kvcache_ref(case.k_new, case.v_new, case.k_cache, case.v_cache, case.slot_mapping)
    out = A.decode_paged(dev.q, dev.k_cache, dev.v_cache, dev.context_lens, dev.block_tables, case.scale)
    torch.cuda.synchronize()
    ref = R.decode_ref(case.q, case.k_cache, case.v_cache, case.context_lens, case.block_tables, case.scale)
    assert_close_to_oracle(out, ref, what)
    assert _lib.read_status() == 0
    return out


def test_cfg1(cuda):
    """8 sequences, contexts in [100,1024], 16 query / 8 KV heads, head_dim 128 (the CPU-runnable
    decode configuration)."""
    _check(cuda, W.cfg1_decode(), "cfg1")


@pytest.mark.parametrize("hq,hkv,d", [(16, 8, 128), (32, 8, 128), (14, 2, 64), (4, 1, 128), (7, 1, 64), (8, 1, 128), (2, 2, 64),
                                      (40, 8, 128), (12, 2, 128), (6, 2, 64)])
def test_geometries(cuda, hq, hkv, d):
    case = W.make_decode_case(11, 6, 1, 1500, hq, hkv, d,
                              context_lens=[1, 255, 256, 257, 1024, 1500])
    _check(cuda, case, f"hq{hq} hkv{hkv} d{d}")


@pytest.mark.parametrize("width", [1, 4, 16, 64])
def test_table_width(cuda, width):
    """The table width is static under CUDA graphs and only bounds the lengths; results must not
    depend on it."""
    lens = [min(200, width * 256), min(width * 256, 3000), 17, width * 256]
    case = W.make_decode_case(12, 4, 1, 1, 16, 8, 128, context_lens=lens, table_width=width)
    _check(cuda, case, f"width{width}")


def test_long_context_split_and_combine(cuda):
    """Qwen2-0.5B geometry, 32768-token contexts in 128 scattered blocks (config 5 shape,
    small batch so the oracle finishes in seconds)."""
    case = W.make_decode_case(13, 3, 1, 1, 14, 2, 64, context_lens=[32768, 20000, 32767])
    _check(cuda, case, "long")


def test_long_context_one_kv_head_per_rank(cuda):
    """The tensor-parallel (2 ranks) shard of the long-context configuration: 7 query heads on 1 KV
    head, head_dim 64, 32768-token contexts."""
    case = W.make_decode_case(23, 3, 1, 1, 7, 1, 64, context_lens=[32768, 32768, 32768])
    _check(cuda, case, "long tp2 shard")


def test_qwen3_8b_geometry_at_8192_tokens(cuda):
    """32 query / 8 KV heads, head_dim 128, contexts up to the 8192 tokens of the decode benchmark."""
    case = W.make_decode_case(24, 5, 1, 1, 32, 8, 128, context_lens=[8192, 2048, 8191, 5000, 4097], table_width=32)
    _check(cuda, case, "8b geometry 8192")


def test_many_short_sequences_share_a_thread_block(cuda):
    """More sequences than threads in a block and far more than thread blocks per KV head: every
    block walks several sequences, a few of them empty, most cut by no range boundary."""
    g = torch.Generator().manual_seed(25)
    lens = torch.randint(0, 200, (300,), generator=g).tolist()
    lens[0] = 0
    lens[-1] = 0
    case = W.make_decode_case(25, 300, 1, 1, 16, 8, 128, context_lens=lens, table_width=4)
    case.slot_mapping.clamp_(min=0)
    dev = case.to(cuda)
    out = A.decode_paged(dev.q, dev.k_cache, dev.v_cache, dev.context_lens, dev.block_tables, case.scale)
    ref = R.decode_ref(case.q, case.k_cache, case.v_cache, case.context_lens, case.block_tables, case.scale)
    assert_close_to_oracle(out, ref, "many short")
    assert _lib.read_status() == 0


def test_one_sequence_spread_over_every_thread_block(cuda):
    """A single long sequence among empty ones: every range holds a piece of it, and the block that
    delivers the last partial merges them all."""
    case = W.make_decode_case(26, 4, 1, 1, 4, 1, 128, context_lens=[0, 30000, 0, 0], table_width=128)
    case.slot_mapping.clamp_(min=0)
    dev = case.to(cuda)
    for _ in range(2):  # the second call finds the counters as the first one left them
        out = A.decode_paged(dev.q, dev.k_cache, dev.v_cache, dev.context_lens, dev.block_tables, case.scale)
    ref = R.decode_ref(case.q, case.k_cache, case.v_cache, case.context_lens, case.block_tables, case.scale)
    assert_close_to_oracle(out, ref, "one long")


@pytest.mark.parametrize("hq,hkv,d", [(16, 8, 128), (32, 8, 128), (14, 2, 64), (4, 1, 128)])
def test_decode_step_equals_store_then_decode(cuda, hq, hkv, d):
    """The one-launch step (store of the new token + decode) must leave the cache exactly as
    store_kvcache does (nanovllm/layers/attention.py:65-66) and give the output of the two
    separate calls; both are compared with the oracle as well."""
    case = W.make_decode_case(27, 9, 1, 1, hq, hkv, d, context_lens=[1, 64, 65, 256, 257, 1000, 1024, 3000, 16],
                              table_width=12)
    sep, fus = case.to(cuda), case.to(cuda)
    A.store_kvcache(sep.k_new, sep.v_new, sep.k_cache, sep.v_cache, sep.slot_mapping)
    expected = A.decode_paged(sep.q, sep.k_cache, sep.v_cache, sep.context_lens, sep.block_tables, case.scale)
    got = A.decode_step(fus.q, fus.k_new, fus.v_new, fus.k_cache, fus.v_cache, fus.slot_mapping, fus.context_lens,
                        fus.block_tables, case.scale)
    torch.cuda.synchronize()
    assert torch.equal(fus.k_cache, sep.k_cache) and torch.equal(fus.v_cache, sep.v_cache)
    assert torch.equal(got, expected)
    R.store_kvcache_ref(case.k_new, case.v_new, case.k_cache, case.v_cache, case.slot_mapping)
    ref = R.decode_ref(case.q, case.k_cache, case.v_cache, case.context_lens, case.block_tables, case.scale)
    assert_close_to_oracle(got, ref, "decode step")
    assert _lib.read_status() == 0


def test_decode_step_slot_rules(cuda):
    """slot < 0: nothing stored, the cached row is used.  A slot that is not the position of the
    newest token: flagged, nothing stored.  Empty rows: nothing stored."""
    case = W.make_decode_case(28, 4, 1, 1, 16, 8, 128, context_lens=[300, 300, 0, 300], table_width=4)
    case.slot_mapping[0] = -1
    case.slot_mapping[1] += 1
    case.slot_mapping[2] = 0
    dev = case.to(cuda)
    k_before, v_before = dev.k_cache.clone(), dev.v_cache.clone()
    _lib.read_status()
    out = A.decode_step(dev.q, dev.k_new, dev.v_new, dev.k_cache, dev.v_cache, dev.slot_mapping, dev.context_lens,
                        dev.block_tables, case.scale)
    torch.cuda.synchronize()
    assert _lib.read_status() == 1  # NVLLM_STATUS_BAD_SLOT, from row 1 only
    s3 = int(case.slot_mapping[3])
    flat_k, flat_kb = dev.k_cache.view(-1, 8, 128), k_before.view(-1, 8, 128)
    assert torch.equal(flat_k[s3], dev.k_new[3]) and torch.equal(dev.v_cache.view(-1, 8, 128)[s3], dev.v_new[3])
    flat_kb[s3] = flat_k[s3]
    v_before.view(-1, 8, 128)[s3] = dev.v_cache.view(-1, 8, 128)[s3]
    assert torch.equal(dev.k_cache, k_before) and torch.equal(dev.v_cache, v_before)  # nothing else was written
    host_k, host_v = dev.k_cache.cpu(), dev.v_cache.cpu()
    ref = R.decode_ref(case.q, host_k, host_v, case.context_lens, case.block_tables, case.scale)
    assert_close_to_oracle(out, ref, "slot rules")


def test_zero_context_rows_and_graph_padding(cuda):
    """Padding rows under graph replay have context_len 0, slot 0 and table row 0
    (nanovllm/engine/model_runner.py:271-280): output rows must be zero, no fault."""
    case = W.make_decode_case(14, 5, 1, 1, 16, 8, 128, context_lens=[300, 0, 0, 513, 0], table_width=16)
    case.block_tables[case.context_lens == 0] = 0
    dev = case.to(cuda)
    out = A.decode_paged(dev.q, dev.k_cache, dev.v_cache, dev.context_lens, dev.block_tables, case.scale)
    ref = R.decode_ref(case.q, case.k_cache, case.v_cache, case.context_lens, case.block_tables, case.scale)
    assert_close_to_oracle(out, ref, "padding")
    assert out[1].abs().max() == 0 and out[4].abs().max() == 0


def test_stale_cache_beyond_context_cannot_leak(cuda):
    """Positions past the context hold NaN/Inf garbage; the output must stay finite."""
    case = W.make_decode_case(15, 3, 1, 1, 16, 8, 128, context_lens=[100, 257, 511])
    for b, n in enumerate(case.context_lens.tolist()):
        blk = int(case.block_tables[b, (n - 1) // 256])
        case.k_cache[blk, n % 256 or 256:] = float("nan")
        case.v_cache[blk, n % 256 or 256:] = float("inf")
    _check(cuda, case, "stale", store_first=False)


def test_bad_block_id_is_flagged_not_dereferenced(cuda):
    case = W.make_decode_case(16, 2, 1, 1, 16, 8, 128, context_lens=[300, 300])
    case.block_tables[1, 1] = 10 ** 6
    dev = case.to(cuda)
    _lib.read_status()
    out = A.decode_paged(dev.q, dev.k_cache, dev.v_cache, dev.context_lens, dev.block_tables, case.scale)
    torch.cuda.synchronize()
    assert _lib.read_status() & 2
    assert torch.isfinite(out.float()).all()


def test_strided_q_and_cuda_graph_replay(cuda):
    """q is a view of the fused qkv activation; the launch is captured once with zeroed
    metadata and replayed with real metadata (nanovllm/engine/model_runner.py:296-336)."""
    hq, hkv, d, B, width = 16, 8, 128, 8, 16
    case = W.make_decode_case(17, B, 100, 3000, hq, hkv, d, table_width=width)
    dev = case.to(cuda)
    qkv = torch.zeros(B, (hq + 2 * hkv) * d, dtype=torch.bfloat16, device=cuda)
    q_view = qkv[:, :hq * d].view(B, hq, d)
    ctx = torch.zeros(B, dtype=torch.int32, device=cuda)
    bt = torch.zeros(B, width, dtype=torch.int32, device=cuda)
    out = torch.zeros(B, hq, d, dtype=torch.bfloat16, device=cuda)
    A.decode_paged(q_view, dev.k_cache, dev.v_cache, ctx, bt, case.scale, out=out)  # warm-up (allocates scratch)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        A.decode_paged(q_view, dev.k_cache, dev.v_cache, ctx, bt, case.scale, out=out)
    q_view.copy_(dev.q)
    ctx.copy_(dev.context_lens)
    bt.copy_(dev.block_tables)
    graph.replay()
    torch.cuda.synchronize()
    ref = R.decode_ref(case.q, case.k_cache, case.v_cache, case.context_lens, case.block_tables, case.scale)
    assert_close_to_oracle(out, ref, "graph replay")
    # replay again with other lengths: the ranges, the pieces and the arrival counters all change
    shorter = (case.context_lens // 3).clamp(min=1)
    ctx.copy_(shorter.to(cuda))
    graph.replay()
    graph.replay()
    torch.cuda.synchronize()
    ref = R.decode_ref(case.q, case.k_cache, case.v_cache, shorter, case.block_tables, case.scale)
    assert_close_to_oracle(out, ref, "graph replay, shorter contexts")


@pytest.mark.parametrize("tp", [2, 4, 8])
def test_head_sharded_ranks_reassemble_the_unsharded_result(cuda, tp):
    """Tensor parallelism: rank r holds query heads [r*Hq/tp, ...) and KV heads [r*Hkv/tp, ...) of
    every cache row (nanovllm/engine/model_runner.py:117, nanovllm/layers/linear.py:141-163) and
    sees identical metadata.  All shards run here on one GPU, one after the other; their outputs
    side by side must match the oracle (and the unsharded kernel's output within rounding: the
    number of ranges, hence where a sequence is cut, depends on the KV heads per rank)."""
    hq, hkv, d = 32, 8, 128
    case = W.make_decode_case(18, 6, 1, 1, hq, hkv, d, context_lens=[700, 1, 2049, 256, 3000, 513], table_width=12)
    dev = case.to(cuda)
    full = A.decode_paged(dev.q, dev.k_cache, dev.v_cache, dev.context_lens, dev.block_tables, case.scale)
    parts = []
    for r in range(tp):
        qs = dev.q[:, r * hq // tp:(r + 1) * hq // tp].contiguous()
        ks = dev.k_cache[:, :, r * hkv // tp:(r + 1) * hkv // tp].contiguous()
        vs = dev.v_cache[:, :, r * hkv // tp:(r + 1) * hkv // tp].contiguous()
        parts.append(A.decode_paged(qs, ks, vs, dev.context_lens, dev.block_tables, case.scale))
    torch.cuda.synchronize()
    ref = R.decode_ref(case.q, case.k_cache, case.v_cache, case.context_lens, case.block_tables, case.scale)
    assert_close_to_oracle(torch.cat(parts, dim=1), ref, f"tp{tp}")
    assert (torch.cat(parts, dim=1).float() - full.float()).abs().max().item() <= 2e-2
