"""Host-side logic that needs no GPU: the layer's contract, the workload generators and the
oracle's own consistency."""
import pytest
import torch

from nano_vllm_b200 import attention as A, context as C, workloads as W
from oracle import paged_attention_ref as R


def test_layer_surface_matches_the_reference_module():
    layer = A.Attention(16, 128, 128 ** -0.5, 8)
    assert (layer.num_heads, layer.head_dim, layer.num_kv_heads) == (16, 128, 8)
    assert layer.k_cache.numel() == 0 and layer.v_cache.numel() == 0  # what allocate_kv_cache looks for
    assert hasattr(layer, "k_cache") and hasattr(layer, "v_cache")
    C.set_context(False, slot_mapping=torch.zeros(1, dtype=torch.int32))
    assert C.get_context().is_prefill is False and C.get_context().block_tables is None
    C.reset_context()
    assert C.get_context().slot_mapping is None


def test_there_is_no_cpu_fallback():
    q = torch.zeros(2, 16, 128, dtype=torch.bfloat16)
    kc = torch.zeros(1, 256, 8, 128, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="CUDA"):
        A.store_kvcache(q[:, :8], q[:, :8], kc, kc, torch.zeros(2, dtype=torch.int32))
    with pytest.raises(RuntimeError, match="CUDA"):
        A.decode_paged(q, kc, kc, torch.ones(2, dtype=torch.int32), torch.zeros(2, 1, dtype=torch.int32), 0.1)
    with pytest.raises(RuntimeError, match="CUDA"):
        cu = torch.tensor([0, 2], dtype=torch.int32)
        A.prefill_varlen(q, q[:, :8], q[:, :8], cu, cu, 2, 2, 0.1)


def test_decode_workload_metadata_is_what_the_runner_would_build():
    case = W.cfg1_decode()
    B = case.q.shape[0]
    assert case.block_tables.dtype == torch.int32 and case.context_lens.dtype == torch.int32
    used = case.block_tables[case.block_tables >= 0]
    assert used.unique().numel() == used.numel(), "physical blocks are not shared between sequences"
    for b in range(B):
        n = int(case.context_lens[b])
        nblk = (n + 255) // 256
        assert (case.block_tables[b, :nblk] >= 0).all() and (case.block_tables[b, nblk:] == -1).all()
        # slot of the token being decoded: last block, last position (model_runner.py:225-229)
        assert int(case.slot_mapping[b]) == int(case.block_tables[b, nblk - 1]) * 256 + (n - 1) % 256
    assert 100 <= int(case.context_lens.min()) and int(case.context_lens.max()) <= 1024


def test_prefill_workload_prefix_sharing_structure():
    case = W.cfg2_prefill()
    lq = (case.cu_seqlens_q[1:] - case.cu_seqlens_q[:-1]).tolist()
    lk = (case.cu_seqlens_k[1:] - case.cu_seqlens_k[:-1]).tolist()
    assert len(lq) == 64 and case.block_tables is not None
    sharers = [i for i in range(64) if lk[i] != lq[i]]
    assert sharers == list(range(3, 64, 4))
    for i in sharers:
        cached = lk[i] - lq[i]
        assert cached % 256 == 0 and 256 <= cached <= 768 and lq[i] >= 1
        nshared = cached // 256
        assert torch.equal(case.block_tables[i, :nshared], case.block_tables[i - 1, :nshared])
    assert case.slot_mapping.numel() == sum(lq) == case.q.shape[0]
    assert case.slot_mapping.unique().numel() == case.slot_mapping.numel()
    assert case.max_seqlen_q == max(lq) and case.max_seqlen_k == max(lk)


def test_oracle_decode_equals_plain_softmax():
    case = W.make_decode_case(51, 3, 1, 1, 4, 2, 64, context_lens=[5, 300, 257])
    out = R.decode_ref(case.q, case.k_cache, case.v_cache, case.context_lens, case.block_tables, case.scale)
    for b in range(3):
        n = int(case.context_lens[b])
        k = R.gather_paged(case.k_cache, case.block_tables[b], n).float()
        v = R.gather_paged(case.v_cache, case.block_tables[b], n).float()
        for h in range(4):
            s = (k[:, h // 2] @ case.q[b, h].float()) * case.scale
            ref = torch.softmax(s, 0) @ v[:, h // 2]
            assert torch.allclose(out[b, h], ref, atol=1e-5, rtol=1e-4)


def test_oracle_prefix_prefill_equals_suffix_of_full_prefill():
    """A sequence with a cached prefix must get the rows a full prefill would give it."""
    case = W.make_prefill_case(52, 2, 1, 1, 4, 2, 64, lengths=[700, 700], shared_blocks=[0, 2])
    R.store_kvcache_ref(case.k, case.v, case.k_cache, case.v_cache, case.slot_mapping)
    out = R.prefill_ref(case.q, case.k_cache, case.v_cache, case.cu_seqlens_q, case.cu_seqlens_k, case.scale,
                        case.block_tables)
    # sequence 1 recomputed from scratch: its K/V = 512 shared rows of sequence 0 + its own 188
    k_full = torch.cat([case.k[:512], case.k[700:]])
    v_full = torch.cat([case.v[:512], case.v[700:]])
    q_full = torch.cat([torch.zeros(512, 4, 64, dtype=torch.bfloat16), case.q[700:]])
    cu = torch.tensor([0, 700], dtype=torch.int32)
    full = R.prefill_ref(q_full, k_full, v_full, cu, cu, case.scale)
    assert torch.allclose(out[700:], full[512:], atol=1e-6)


def test_algorithmic_work_formulas():
    assert W.decode_bytes([256, 1], 16, 8, 128) == 257 * 8 * 128 * 4 + 2 * 2 * 16 * 128 * 2 + 4 * (2 + 2)
    assert W.store_bytes(10, 1024) == 10 * 1024 * 8 + 40
    assert W.prefill_flops([3], [3], 1, 1) == 4 * 6
    assert W.prefill_flops([2], [258], 2, 64) == 4 * 2 * 64 * (2 * 256 + 3)


def test_when_the_peer_memory_all_reduce_is_preferred():
    """Decode-sized tensors go to the peer kernel, prefill-sized ones to the library collective."""
    from nano_vllm_b200.allreduce import prefer_peer_kernel as prefer
    mb = 8 << 20
    assert prefer(256 * 1024 * 2, 2, mb) and prefer(256 * 4096 * 2, 2, mb) and prefer(4 << 20, 2, mb)
    assert not prefer(16384 * 1024 * 2, 2, mb)            # a 16k-token prefill batch: 32 MiB
    assert prefer(256 * 1024 * 2, 4, mb) and prefer(256 * 1024 * 2, 8, mb)
    assert prefer(256 * 4096 * 2, 4, mb) and prefer(256 * 4096 * 2, 8, mb)
    assert not prefer(0, 2, mb)


def test_all_reduce_protocol_choice_is_host_arithmetic(lib):
    """Cells for small tensors, two shots for larger ones at more than two ranks, one shot at two
    ranks and for tensors with a ragged tail; a forced protocol that does not apply falls back."""
    from nano_vllm_b200.allreduce import protocol_for
    mb = 8 << 20
    assert protocol_for(32 << 10, 2, mb) == "cells" and protocol_for(2 << 20, 2, mb) == "cells"
    assert protocol_for(4 << 20, 2, mb) == "one-shot"
    assert protocol_for(32 << 10, 8, mb) == "cells" and protocol_for(128 << 10, 8, mb) == "cells"
    assert protocol_for(512 << 10, 4, mb) == "cells" and protocol_for(1 << 20, 4, mb) == "cells-two-shot"
    assert protocol_for(512 << 10, 8, mb) == "cells" and protocol_for(1 << 20, 8, mb) == "cells-two-shot"
    assert protocol_for(2 << 20, 4, mb) == "cells-two-shot" and protocol_for(2 << 20, 8, mb) == "cells-two-shot"
    assert protocol_for(2 << 20, 8, mb, forced=3) == "two-shot" and protocol_for(6 << 20, 4, mb) == "two-shot"
    assert protocol_for((2 << 20) + 6, 8, mb) == "cells-two-shot"    # a ragged tail is fine for cells
    assert protocol_for(2 << 20, 8, mb, forced=2) == "one-shot"
    assert protocol_for(2 << 20, 2, mb, forced=3) == "cells"           # two shots need more than two ranks
    assert protocol_for(2 << 20, 8, mb, forced=1) == "cells-two-shot"  # cells to every peer do not fit: 2 x 2 MiB x 8 > 8 MiB


def test_fused_projection_tile_choice_is_host_arithmetic(lib):
    """Tile width of the projection fused with its all-reduce: the narrowest of 32 / 64 / 128 columns
    that leaves one tile per thread block (128 blocks), 0 for shapes the kernel refuses."""
    mb = 8 << 20
    assert lib.nvllm_ar_gemm_tile(16, 4096, 512, 8, mb) == 32
    assert lib.nvllm_ar_gemm_tile(256, 4096, 1536, 8, mb) == 64
    assert lib.nvllm_ar_gemm_tile(512, 4096, 512, 8, mb) == 128
    assert lib.nvllm_ar_gemm_tile(256, 1024, 1024, 2, mb) == 32
    assert lib.nvllm_ar_gemm_tile(1024, 4096, 512, 8, mb) == 0   # cell areas too small
    assert lib.nvllm_ar_gemm_tile(256, 4096, 512, 8, 1 << 20) == 0
    assert lib.nvllm_ar_gemm_tile(8, 4096, 100, 2, mb) == 0      # k not a multiple of 8
    assert lib.nvllm_ar_gemm_tile(8, 48, 64, 2, mb) == 0         # n not a multiple of 32
    assert lib.nvllm_ar_gemm_tile(8, 4096, 512, 9, mb) == 0      # more ranks than the areas have regions for


def test_oracle_row_parallel_projection_rounds_every_rank_once():
    """The oracle's partials are bf16 (what each rank's GEMM returns), not fp32: the sum of rounded
    partials differs from the rounded product over the whole k."""
    g = torch.Generator().manual_seed(3)
    xs = [torch.randn(4, 64, generator=g).to(torch.bfloat16) for _ in range(4)]
    ws = [torch.randn(32, 64, generator=g).to(torch.bfloat16) for _ in range(4)]
    got = R.row_parallel_linear_ref(xs, ws)
    partials = [(x.float() @ w.float().t()).to(torch.bfloat16) for x, w in zip(xs, ws)]
    assert torch.equal(got, R.allreduce_ref(partials))
    whole = (torch.cat(xs, 1).float() @ torch.cat(ws, 1).float().t()).to(torch.bfloat16)
    assert got.shape == whole.shape and not torch.equal(got, whole)
    assert float((got.float() - whole.float()).abs().max()) <= 4 * 2.0 ** -8 * float(whole.float().abs().max())
