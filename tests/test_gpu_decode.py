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
    """BASELINE config 1: 8 sequences, ctx in [100,1024], 16q/8kv heads, D=128."""
    _check(cuda, W.cfg1_decode(), "cfg1")


@pytest.mark.parametrize("hq,hkv,d", [(16, 8, 128), (32, 8, 128), (14, 2, 64), (4, 1, 128), (7, 1, 64), (8, 1, 128), (2, 2, 64),
                                      (40, 8, 128), (12, 2, 128), (6, 2, 64)])
def test_geometries(cuda, hq, hkv, d):
    case = W.make_decode_case(11, 6, 1, 1500, hq, hkv, d,
                              context_lens=[1, 255, 256, 257, 1024, 1500])
    _check(cuda, case, f"hq{hq} hkv{hkv} d{d}")


@pytest.mark.parametrize("width", [1, 4, 16, 64])
def test_table_width_changes_split_plan(cuda, width):
    """The split-KV plan depends on the table width (static under CUDA graphs), not on the
    lengths; results must not."""
    lens = [min(200, width * 256), min(width * 256, 3000), 17, width * 256]
    case = W.make_decode_case(12, 4, 1, 1, 16, 8, 128, context_lens=lens, table_width=width)
    _check(cuda, case, f"width{width}")


def test_long_context_split_and_combine(cuda):
    """Qwen2-0.5B geometry, 32768-token contexts in 128 scattered blocks (config 5 shape,
    small batch so the oracle finishes in seconds)."""
    case = W.make_decode_case(13, 3, 1, 1, 14, 2, 64, context_lens=[32768, 20000, 32767])
    chunk, splits = _lib.decode_plan(3, 128, 14, 2, 64)
    assert splits > 1
    _check(cuda, case, "long")


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


@pytest.mark.parametrize("tp", [2, 4, 8])
def test_head_sharded_ranks_reassemble_the_unsharded_result(cuda, tp):
    """Tensor parallelism: rank r holds query heads [r*Hq/tp, ...) and KV heads [r*Hkv/tp, ...) of
    every cache row (nanovllm/engine/model_runner.py:117, nanovllm/layers/linear.py:141-163) and
    sees identical metadata.  All shards run here on one GPU, one after the other; their outputs
    side by side must equal the unsharded kernel's output bit for bit (same arithmetic per head)
    and match the oracle."""
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
    # per-head arithmetic does not depend on how many heads share the launch as long as the split
    # plan is the same; the plan depends on batch*Hkv, so compare against the oracle above and
    # check exact equality only where the plans agree
    if _lib.decode_plan(6, 12, hq // tp, hkv // tp, d) == _lib.decode_plan(6, 12, hq, hkv, d):
        assert torch.equal(torch.cat(parts, dim=1), full)
