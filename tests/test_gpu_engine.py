"""The unmodified nano-vllm engine (installed copy under baseline/_ref; skipped when absent) with
the B200 attention layer swapped in: generate() with CUDA graphs, then the same prompts again so
that the block manager serves their prefixes from the cache and the prefill reads them through
block_tables."""
import json
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
REF = ROOT / "baseline" / "_ref"

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not (REF / "nanovllm").is_dir(), reason="no nano-vllm install under baseline/_ref")]

SCRIPT = r"""
import json, os, random, sys, tempfile
sys.path.insert(0, %(root)r)
from nano_vllm_b200 import e2e, _lib
os.chdir(tempfile.mkdtemp())
e2e.GEOMETRY["tiny"] = dict(hidden_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                            head_dim=128, intermediate_size=512, tie_word_embeddings=True)
llm = e2e.make_engine(e2e.write_model_dir("tiny"), %(attn)r, %(ref)r, enforce_eager=False, max_model_len=2048,
                      max_num_seqs=16, tensor_parallel_size=%(tp)d)
from nanovllm.sampling_params import SamplingParams
random.seed(1)
prompts = [[random.randint(0, 151935) for _ in range(n)] for n in (300, 700, 257, 1100, 90)]
sp = SamplingParams(temperature=0.0, max_tokens=40, ignore_eos=True)
first = llm.generate(prompts, sp, use_tqdm=False)
hits_before = sum(1 for b in llm.scheduler.block_manager.blocks if b.hash != -1)
second = llm.generate(prompts, sp, use_tqdm=False)   # full blocks of every prompt are now cached
same = sum(a == b for x, y in zip(first, second) for a, b in zip(x["token_ids"], y["token_ids"]))
total = sum(len(x["token_ids"]) for x in first)
print(json.dumps({"lens": [len(x["token_ids"]) for x in first + second], "same": same, "total": total,
                  "tokens": [x["token_ids"] for x in first + second],
                  "cached_blocks": hits_before, "status": _lib.read_status(), "launches": _lib.launch_count()}))
"""


def _run(attn, tp=1):
    code = SCRIPT % {"root": str(ROOT), "ref": str(REF), "attn": attn, "tp": tp}
    proc = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600, cwd=str(ROOT))
    assert proc.returncode == 0, proc.stderr[-3000:]
    return json.loads([ln for ln in proc.stdout.splitlines() if ln.startswith("{")][-1])


def test_generate_with_graphs_and_prefix_cache():
    d = _run("b200-fused")
    assert d["lens"] == [40] * 10
    assert d["cached_blocks"] >= 8            # 1 + 2 + 1 + 4 full blocks of the first pass were hashed
    assert d["status"] == 0 and d["launches"] > 0
    # greedy decoding: the second pass (prefix read through block_tables) must reproduce the first
    # (packed prefill) up to rare bf16 near-ties in a random-weight model
    assert d["same"] >= 0.9 * d["total"], d


def test_one_launch_decode_inputs_and_fused_sampler_change_no_greedy_token():
    """With temperature 0 the engine is deterministic: staging the decode inputs through one copy
    and one launch, and taking the argmax in the sampling kernel, must reproduce every token of
    the run that uses the engine's own prepare_decode / run_model / Sampler."""
    stock_path, fused_path = _run("b200-fused"), _run("b200-full")
    assert fused_path["status"] == 0 and fused_path["lens"] == [40] * 10
    assert fused_path["tokens"] == stock_path["tokens"]


def _gpus():
    import torch
    return torch.cuda.device_count()


@pytest.mark.skipif(_gpus() < 2, reason="needs two GPUs")
def test_tensor_parallel_engine_with_every_optional_step():
    """Two ranks (rank 0 plus a spawned worker that receives pickled sequences without sampling
    parameters): head-sharded attention, fused pre-attention, one-launch decode inputs on both
    ranks, the sampler on rank 0, and the peer-memory all-reduce behind both row-parallel
    projections, with decode graphs captured around them."""
    d = _run("b200-full-ar", tp=2)
    assert d["lens"] == [40] * 10 and d["status"] == 0 and d["launches"] > 0
    assert d["same"] >= 0.9 * d["total"], d
    # The vocabulary-sharded sampling tail (every rank reduces its slice of the logits to one
    # candidate per row, 8 bytes per row are merged) must pick the tokens that rank 0 picks from
    # the gathered and concatenated logits: greedy decoding, so token for token.  The two runs
    # differ in the all-reduce as well (peer kernel and NCCL both sum in fp32, in rank order at
    # two ranks), so a rare bf16 near-tie may still flip a token: nearly all must agree.
    g = _run("b200-full", tp=2)
    same = sum(a == b for x, y in zip(d["tokens"], g["tokens"]) for a, b in zip(x, y))
    assert same >= 0.95 * d["total"] * 2, (same, d["total"])
