"""Installs the B200 attention layer into an importable nano-vllm without editing its tree.

``install()`` registers a module named ``nanovllm.layers.attention`` that exports the same two
names the reference module exports (``Attention``, ``store_kvcache``;
nanovllm/layers/attention.py:32-79) and makes the layer read nano-vllm's own per-step context
(nanovllm/utils/context.py:16-17).  Call it before ``nanovllm.models`` is imported (i.e. before
``from nanovllm import LLM``), because the model files bind ``Attention`` at import time
(nanovllm/models/qwen3.py:8).

Optional steps after ``install()``, each replacing one method of the engine by a version that
calls this package: ``fuse_pre_attention()`` (q/k norm + rotary + KV store in one launch),
``fuse_sampler()`` (one-pass token sampling), ``fuse_decode_inputs()`` (decode-step inputs in
one copy and one launch) and, for tensor-parallel runs, ``fuse_all_reduce()`` (peer-memory sum
behind the row-parallel projections) and ``fuse_lm_head()`` (every rank samples its own slice of
the vocabulary; 8 bytes per row travel instead of the logits).
"""
from __future__ import annotations

import importlib
import sys
import types

from . import attention as _attention

MODULE_NAME = "nanovllm.layers.attention"


def _fused_attention_forward(has_qk_norm: bool):
    """Replacement for Qwen3Attention.forward / Qwen2Attention.forward
    (nanovllm/models/qwen3.py:77-113, qwen2.py:77-97): same projections, but q/k norm, rotary
    embedding and the KV-cache store run as one launch on the fused qkv activation."""

    def forward(self, positions, hidden_states):
        qkv = self.qkv_proj(hidden_states)
        attn = self.attn
        ctx = _attention._get_context()
        _attention.qk_norm_rope_store(
            qkv, positions,
            self.q_norm.weight if has_qk_norm else None, self.k_norm.weight if has_qk_norm else None,
            self.rotary_emb.cos_sin_cache, self.q_norm.eps if has_qk_norm else 0.0,
            ctx.slot_mapping, attn.k_cache, attn.v_cache, self.num_heads, self.num_kv_heads, self.head_dim)
        q, k, v = qkv.split([self.q_size, self.kv_size, self.kv_size], dim=-1)
        return self.o_proj(attn(q, k, v, kv_stored=True))

    return forward


def fuse_pre_attention() -> None:
    """Optional second step after ``install()``: also replace the q/k-norm + rotary + store
    sequence of nano-vllm's Qwen3 and Qwen2 attention blocks by the fused kernel."""
    qwen3 = importlib.import_module("nanovllm.models.qwen3")
    qwen2 = importlib.import_module("nanovllm.models.qwen2")
    qwen3.Qwen3Attention.forward = _fused_attention_forward(True)
    qwen2.Qwen2Attention.forward = _fused_attention_forward(False)


def fuse_sampler(seed: int | None = None) -> None:
    """Optional step: replace ``Sampler.forward`` (nanovllm/layers/sampler.py:10-26) by the
    one-pass sampling kernel.  Greedy rows (temperature 0) give the reference's tokens; sampled
    rows follow the same distribution but another random stream (Philox keyed by ``seed``,
    default ``torch.initial_seed()``, counted by the number of calls), so they are not the
    tokens the reference's ``exponential_`` stream would have picked."""
    sampler = importlib.import_module("nanovllm.layers.sampler")
    import torch
    state = {"seed": torch.initial_seed() if seed is None else seed, "step": 0}

    def forward(self, logits, temperatures):
        state["step"] += 1
        return _attention.sample_tokens(logits, temperatures, seed=state["seed"], step=state["step"])

    sampler.Sampler.forward = forward


# What the replacement of ModelRunner.run does; switched on by fuse_decode_inputs / fuse_lm_head.
_runner = {"decode_inputs": False, "lm_head": False, "seed": 0, "step": 0, "stock_run": None}


def _run(self, seqs, is_prefill, temperatures_list=None):
    """ModelRunner.run (nanovllm/engine/model_runner.py:284-293) with the optional steps.  Rank 0 of
    a tensor-parallel engine passes the step's temperatures along with the sequences when the
    LM-head step is on (the pickled sequences carry no sampling parameters, sequence.py:74-76)."""
    import torch
    import torch.distributed as dist
    ctx = importlib.import_module("nanovllm.utils.context")
    lm = _runner["lm_head"] and self.world_size > 1
    graphs = getattr(self, "graphs", None)
    staged = (_runner["decode_inputs"] and not is_prefill and not self.enforce_eager and bool(graphs)
              and len(seqs) <= self.graph_bs[-1])
    if not staged and not lm:
        return _runner["stock_run"](self, seqs, is_prefill)
    if lm and temperatures_list is None:
        temperatures_list = [seq.temperature for seq in seqs]  # rank 0
    with torch.inference_mode():
        if staged:
            from .decode_inputs import DecodeInputStager
            gv = self.graph_vars
            stager = getattr(self, "_nvllm_stager", None)
            if stager is None:
                rows, width = gv["block_tables"].shape
                stager = self._nvllm_stager = DecodeInputStager(rows, width, gv["block_tables"].device)
            bs = len(seqs)
            graph_bs = next(x for x in self.graph_bs if x >= bs)
            temperatures = stager.stage(seqs, graph_bs, gv, temperatures=temperatures_list if lm else None,
                                        with_temperatures=lm or self.rank == 0)
            ctx.set_context(False, slot_mapping=gv["slot_mapping"][:bs], context_lens=gv["context_lens"][:bs],
                            block_tables=gv["block_tables"][:bs])
            graphs[graph_bs].replay()
            logits = self.model.compute_logits(gv["outputs"][:bs])
        else:
            input_ids, positions = self.prepare_prefill(seqs) if is_prefill else self.prepare_decode(seqs)
            temperatures = torch.tensor(temperatures_list, dtype=torch.float32, pin_memory=True).cuda(non_blocking=True)
            logits = self.run_model(input_ids, positions, is_prefill)
        if lm:
            # every rank reduces its slice of the vocabulary to one candidate per row; a MAX over the
            # ranks of 8 bytes per row replaces the gather + cat of the logits
            _runner["step"] += 1
            cand = _attention.sample_candidates(logits, temperatures, self.rank * logits.shape[1],
                                                seed=_runner["seed"], step=_runner["step"])
            dist.reduce(cand, dst=0, op=dist.ReduceOp.MAX)
            token_ids = _attention.sample_unpack(cand).tolist() if self.rank == 0 else None
        else:
            token_ids = self.sampler(logits, temperatures).tolist() if self.rank == 0 else None
    ctx.reset_context()
    return token_ids


def _install_run() -> None:
    mr = importlib.import_module("nanovllm.engine.model_runner")
    if _runner["stock_run"] is None:
        _runner["stock_run"] = mr.ModelRunner.run
        mr.ModelRunner.run = _run


def fuse_decode_inputs() -> None:
    """Optional step: decode steps that replay a CUDA graph get their inputs through one staged
    copy and one launch (decode_inputs.DecodeInputStager) instead of ``prepare_decode`` /
    ``prepare_sample`` and the clear-and-copy in ``run_model``
    (nanovllm/engine/model_runner.py:218-258, 271-282).  Prefill steps, eager decode and batches
    beyond the captured sizes go through the stock ``ModelRunner.run``."""
    _install_run()
    _runner["decode_inputs"] = True


def fuse_lm_head(seed: int = 0x5EED) -> None:
    """Optional step for tensor-parallel runs: ``ParallelLMHead.forward``
    (nanovllm/layers/embed_head.py:68-88) keeps every rank's slice of the logits where it is (no
    ``dist.gather`` of ``[batch, vocab / ranks]`` per rank, no ``torch.cat`` on rank 0); every rank
    runs the one-pass sampler over its slice (``sample_candidates``) and the ranks' candidates are
    merged by one 8-byte-per-row MAX reduction.  Rank 0 sends the step's temperatures along with
    the sequences (``ModelRunner.call``), since the workers' copies of the sequences carry none.
    With one rank nothing changes.  Sampled rows use the generator of ``fuse_sampler`` keyed by
    ``seed`` and counted by the number of steps, the same on every rank; greedy rows give the
    reference's tokens."""
    import torch.nn.functional as F
    embed_head = importlib.import_module("nanovllm.layers.embed_head")
    mr = importlib.import_module("nanovllm.engine.model_runner")
    ctx = importlib.import_module("nanovllm.utils.context")
    _install_run()
    _runner["lm_head"] = True
    _runner["seed"] = seed
    stock_forward = embed_head.ParallelLMHead.forward
    stock_call = mr.ModelRunner.call

    def forward(self, x):
        if self.tp_size == 1:
            return stock_forward(self, x)
        context = ctx.get_context()
        if context.is_prefill:  # only each sequence's last position is sampled (embed_head.py:72-74)
            x = x[context.cu_seqlens_q[1:] - 1].contiguous()
        return F.linear(x, self.weight, self.bias)  # this rank's slice of the vocabulary

    def call(self, method_name, *args):
        if method_name == "run" and self.world_size > 1 and self.rank == 0 and len(args) == 2:
            args = (*args, [seq.temperature for seq in args[0]])
        return stock_call(self, method_name, *args)

    embed_head.ParallelLMHead.forward = forward
    mr.ModelRunner.call = call


FUSED_GEMM_MAX_TOKENS = 512  # the decode graphs' largest batch (model_runner.py:306)


def fuse_all_reduce(max_bytes: int = 8 << 20, wait_ms: int = 60000, fuse_gemm: bool = False) -> None:
    """Optional step for tensor-parallel runs: ``RowParallelLinear.forward``
    (nanovllm/layers/linear.py:195-199) sums its partial outputs with the peer-memory kernel
    (allreduce.PeerAllReduce) where that is expected to be the faster one (decode-sized tensors;
    see PeerAllReduce.preferred), and with ``dist.all_reduce`` otherwise (prefill-sized tensors).  The peer mapping is made at the first
    call outside stream capture, which every rank reaches at the same point (the engine's warm-up
    forward).  Ranks of the engine run loosely coupled (a worker can be seconds behind while it
    compiles or captures), hence the long default wait.  A wait that does run out leaves a latch
    in the kernel's buffers (later calls no longer wait and their sums are wrong) that only a
    shutdown clears; every 256th eager call (prefill steps) therefore reads the device status
    word and raises if the time-out bit is set, instead of generating on.  With ``fuse_gemm`` a
    bias-free projection of a decode-sized batch runs as ONE launch that multiplies and sums
    (PeerAllReduce.linear_all_reduce) where its shape allows."""
    import torch
    import torch.distributed as dist
    import torch.nn.functional as F
    linear = importlib.import_module("nanovllm.layers.linear")
    from . import _lib
    from .allreduce import PeerAllReduce
    state = {"ar": None, "eager_calls": 0}

    def forward(self, x):
        if self.tp_size == 1:
            return F.linear(x, self.weight, self.bias)
        ar = state["ar"]
        capturing = torch.cuda.is_current_stream_capturing()
        if ar is None and not capturing:
            ar = state["ar"] = PeerAllReduce(dist.get_rank(), dist.get_world_size(), max_bytes, wait_ms=wait_ms)
        if ar is not None and not capturing:
            state["eager_calls"] += 1
            if state["eager_calls"] % 256 == 0 and _lib.read_status() & 4:
                raise RuntimeError("nano_vllm_b200: a peer all-reduce gave up waiting for another rank "
                                   "(NVLLM_STATUS_TIMEOUT); the sums since then are invalid")
        if (fuse_gemm and ar is not None and self.bias is None and x.dim() == 2 and x.shape[0] <= FUSED_GEMM_MAX_TOKENS
                and ar.linear_fits(x, self.weight)):
            return ar.linear_all_reduce(x, self.weight)
        y = F.linear(x, self.weight, self.bias if self.tp_rank == 0 else None)
        if ar is not None and ar.preferred(y):
            ar.all_reduce(y)
        else:
            dist.all_reduce(y)
        return y

    linear.RowParallelLinear.forward = forward


def install() -> types.ModuleType:
    already = sys.modules.get(MODULE_NAME)
    if already is not None and getattr(already, "__nano_vllm_b200__", False):
        return already
    if already is not None or any(m in sys.modules for m in ("nanovllm.models.qwen3", "nanovllm.models.qwen2")):
        raise RuntimeError("install() must run before anything of nanovllm is imported: importing the "
                           "package pulls in its models, which bind Attention at import time")
    mod = types.ModuleType(MODULE_NAME)
    mod.__doc__ = "nano-vllm attention layer backed by libnvllm_b200.so"
    mod.Attention = _attention.Attention
    mod.store_kvcache = _attention.store_kvcache
    mod.__nano_vllm_b200__ = True
    sys.modules[MODULE_NAME] = mod  # registered first: `import nanovllm` below already imports the models
    ctx = importlib.import_module("nanovllm.utils.context")
    _attention.use_context_getter(ctx.get_context)
    mod.get_context = ctx.get_context
    layers = sys.modules.get("nanovllm.layers")
    if layers is not None:
        setattr(layers, "attention", mod)
    for name in ("nanovllm.models.qwen3", "nanovllm.models.qwen2"):
        m = sys.modules.get(name)
        if m is not None and getattr(m, "Attention", None) is not _attention.Attention:
            raise RuntimeError(f"{name} bound another Attention class; the swap did not take effect")
    return mod
