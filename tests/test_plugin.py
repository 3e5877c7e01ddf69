"""The import-time swap of nano-vllm's attention layer (plugin.install) against an installed
copy of the reference (baseline/_ref, made with pip --target; skipped when it is absent).
Runs in child processes because the swap must happen before anything of nanovllm is imported."""
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
REF = ROOT / "baseline" / "_ref"

pytestmark = pytest.mark.skipif(not (REF / "nanovllm").is_dir(), reason="no nano-vllm install under baseline/_ref")


def _run(code: str) -> str:
    proc = subprocess.run([sys.executable, "-c", code], cwd=str(ROOT), capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stderr[-2000:]
    return proc.stdout.strip().splitlines()[-1]


PRELUDE = f"import sys; sys.path.insert(0, {str(REF)!r}); sys.path.insert(0, {str(ROOT)!r})\n"


def test_install_replaces_the_layer_the_models_bind():
    out = _run(PRELUDE + """
from nano_vllm_b200 import plugin, attention
plugin.install()
import nanovllm.models.qwen3 as q3, nanovllm.models.qwen2 as q2
from nanovllm.utils.context import set_context, get_context
import nanovllm.layers.attention as mod
assert q3.Attention is attention.Attention and q2.Attention is attention.Attention
assert mod.store_kvcache is attention.store_kvcache
set_context(True, max_seqlen_q=7)
assert attention._get_context().max_seqlen_q == 7      # the layer reads the engine's own context
assert "flash_attn" not in sys.modules                  # the attention path no longer imports it
print("ok")
""")
    assert out == "ok"


def test_install_refuses_to_run_after_the_models_were_imported():
    out = _run(PRELUDE + """
import nanovllm                      # binds the stock layer
from nano_vllm_b200 import plugin
try:
    plugin.install()
    print("no error")
except RuntimeError as e:
    print("refused")
""")
    assert out == "refused"


def test_fuse_pre_attention_swaps_the_attention_blocks_forward():
    out = _run(PRELUDE + """
from nano_vllm_b200 import plugin
plugin.install()
import nanovllm.models.qwen3 as q3, nanovllm.models.qwen2 as q2
before = q3.Qwen3Attention.forward
plugin.fuse_pre_attention()
assert q3.Qwen3Attention.forward is not before and q2.Qwen2Attention.forward.__name__ == "forward"
print("ok")
""")
    assert out == "ok"


def test_optional_steps_replace_exactly_one_method_each():
    out = _run(PRELUDE + """
from nano_vllm_b200 import plugin
plugin.install()
import nanovllm.layers.sampler as sampler, nanovllm.layers.linear as linear, nanovllm.engine.model_runner as mr
before = (sampler.Sampler.forward, mr.ModelRunner.run, linear.RowParallelLinear.forward)
keep = (mr.ModelRunner.prepare_prefill, mr.ModelRunner.run_model, linear.ColumnParallelLinear.forward)
plugin.fuse_sampler(seed=1)
plugin.fuse_decode_inputs()
plugin.fuse_all_reduce()
after = (sampler.Sampler.forward, mr.ModelRunner.run, linear.RowParallelLinear.forward)
assert all(a is not b for a, b in zip(after, before))
assert keep == (mr.ModelRunner.prepare_prefill, mr.ModelRunner.run_model, linear.ColumnParallelLinear.forward)
# without a GPU nothing of the package can run: the replaced method must fail loudly, not fall back
import torch
if not torch.cuda.is_available():
    try:
        sampler.Sampler().forward(torch.zeros(2, 8), torch.zeros(2))
        print("fell back")
    except (AssertionError, RuntimeError, ImportError):
        print("ok")
else:
    print("ok")
""")
    assert out == "ok"


def test_lm_head_step_sends_the_temperatures_to_the_worker_ranks():
    """The sequences that reach a worker rank are pickled without sampling parameters
    (nanovllm/engine/sequence.py:74-76); with the vocabulary-sharded sampling step every rank
    samples, so rank 0's call("run", seqs, is_prefill) must carry the step's temperatures, and the
    LM head must keep its slice of the logits instead of gathering."""
    out = _run(PRELUDE + """
from nano_vllm_b200 import plugin
plugin.install()
import torch, types
import nanovllm.engine.model_runner as mr, nanovllm.layers.embed_head as eh
from nanovllm.utils.context import set_context
stock_forward, stock_call, stock_run = eh.ParallelLMHead.forward, mr.ModelRunner.call, mr.ModelRunner.run
plugin.fuse_lm_head(seed=7)
assert eh.ParallelLMHead.forward is not stock_forward and mr.ModelRunner.call is not stock_call
assert mr.ModelRunner.run is not stock_run
# rank 0 of two: the message to the workers and the local call both get the temperatures
runner = object.__new__(mr.ModelRunner)
runner.world_size, runner.rank = 2, 0
sent, ran = [], []
runner.write_shm = lambda name, *args: sent.append((name, args))
runner.run = lambda *args: ran.append(args) or "tokens"
seqs = [types.SimpleNamespace(temperature=0.0), types.SimpleNamespace(temperature=0.6)]
assert runner.call("run", seqs, False) == "tokens"
assert sent == [("run", (seqs, False, [0.0, 0.6]))] and ran == [(seqs, False, [0.0, 0.6])]
# other methods and single-rank runs are passed through untouched
runner.exit = lambda: "bye"
assert runner.call("exit") == "bye" and sent[-1] == ("exit", ())
runner.world_size = 1
assert runner.call("run", seqs, True) == "tokens" and ran[-1] == (seqs, True)
# the head keeps its slice: no gather, last rows only under prefill
head = object.__new__(eh.ParallelLMHead)
torch.nn.Module.__init__(head)
head.tp_size, head.tp_rank = 2, 1
head.weight = torch.nn.Parameter(torch.randn(6, 4))
head.bias = None
x = torch.randn(5, 4)
set_context(True, cu_seqlens_q=torch.tensor([0, 2, 5], dtype=torch.int32))
y = head(x)
assert y.shape == (2, 6) and torch.allclose(y, x[[1, 4]] @ head.weight.T)
set_context(False)
assert head(x).shape == (5, 6)
print("ok")
""")
    assert out == "ok"


def test_row_parallel_forward_picks_the_fused_projection_only_where_it_applies():
    """RowParallelLinear.forward after fuse_all_reduce(fuse_gemm=True): a bias-free projection of at
    most 512 tokens whose shape the kernel takes goes through ONE call (product + sum); a bias, a
    larger batch or a refused shape use F.linear followed by the peer sum (small tensors) or
    dist.all_reduce (large ones); without fuse_gemm the fused call is never made."""
    out = _run(PRELUDE + """
from nano_vllm_b200 import plugin, allreduce as AR
plugin.install()
import torch, torch.distributed as dist
import nanovllm.layers.linear as linear
calls = []
class FakeAR:
    def __init__(self, rank, world, max_bytes, wait_ms=None):
        calls.append(("init", rank, world))
    def linear_fits(self, x, w):
        return x.shape[1] % 8 == 0
    def linear_all_reduce(self, x, w):
        calls.append(("fused", tuple(x.shape)))
        return x @ w.t()
    def preferred(self, y):
        return y.numel() <= 4096
    def all_reduce(self, y):
        calls.append(("peer", tuple(y.shape)))
        return y
AR.PeerAllReduce = FakeAR
dist.get_rank, dist.get_world_size = (lambda: 1), (lambda: 2)
dist.all_reduce = lambda y: calls.append(("nccl", tuple(y.shape)))
torch.cuda.is_current_stream_capturing = lambda: False
def layer(k, n, bias):
    m = object.__new__(linear.RowParallelLinear)
    torch.nn.Module.__init__(m)
    m.tp_size, m.tp_rank = 2, 1
    m.weight = torch.nn.Parameter(torch.randn(n, k))
    m.bias = torch.nn.Parameter(torch.randn(n)) if bias else None
    return m
plugin.fuse_all_reduce(fuse_gemm=True)
x = torch.randn(16, 64)
y = layer(64, 32, False)(x)
assert calls == [("init", 1, 2), ("fused", (16, 64))] and y.shape == (16, 32)
del calls[:]
layer(64, 32, True)(x)                       # bias: unfused, small -> peer sum
layer(64, 32, False)(torch.randn(600, 64))   # more than 512 tokens: unfused, large -> NCCL
layer(60, 32, False)(torch.randn(16, 60))    # shape the kernel refuses
assert calls == [("peer", (16, 32)), ("nccl", (600, 32)), ("peer", (16, 32))], calls
del calls[:]
plugin.fuse_all_reduce()
layer(64, 32, False)(x)
assert calls == [("init", 1, 2), ("peer", (16, 32))], calls
one = layer(64, 32, True)
one.tp_size, one.tp_rank = 1, 0
del calls[:]
assert torch.allclose(one(x), x @ one.weight.t() + one.bias) and calls == []
print("ok")
""")
    assert out == "ok"
