"""End-to-end throughput of nano-vllm with the B200 attention layer plugged in.

    python -m nano_vllm_b200.e2e [--attn b200|b200-fused|b200-full|reference] [--tp N] [--model qwen3-0.6b|qwen3-8b]
                                 [--num-seqs 256] [--ref-path baseline/_ref]

Runs the reference engine UNMODIFIED (scheduler, block manager with prefix caching, model
runner, CUDA-graph capture, tensor-parallel workers) from an installed copy of nano-vllm and
swaps only ``nanovllm.layers.attention`` (see plugin.py).  The workload is the reference's
own benchmark (its bench.py:9-28): ``--num-seqs`` requests of random token ids, prompt and
output lengths uniform in [100, 1024], temperature 0.6, ignore_eos; throughput = generated
tokens / wall time of ``generate`` after one warm-up request, prefill included.

No checkpoint or tokenizer is needed: weights are random-initialised in place (N(0, 0.02),
norm weights 1) instead of being read from safetensors, and prompts are token ids.  Three
small shims make the unmodified engine run in this environment; none touches the attention
path: (1) ``hf_config.rope_scaling`` is reset to None (transformers >= 5 fills it with a
default dict that the engine's ``get_rope`` rejects); (2) ``load_model`` is replaced by the
random initialiser; (3) the tokenizer is a stub (ids in, ids out).
"""
from __future__ import annotations

import argparse
import atexit
import json
import os
import random
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]

GEOMETRY = {
    # hidden, layers, q heads, kv heads, head_dim, intermediate (nano-vllm models/qwen3_06b.txt:10-29)
    "qwen3-0.6b": dict(hidden_size=1024, num_hidden_layers=28, num_attention_heads=16, num_key_value_heads=8,
                       head_dim=128, intermediate_size=3072, tie_word_embeddings=True),
    "qwen3-8b": dict(hidden_size=4096, num_hidden_layers=36, num_attention_heads=32, num_key_value_heads=8,
                     head_dim=128, intermediate_size=12288, tie_word_embeddings=False),
}


def write_model_dir(name: str) -> str:
    cfg = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=151936, hidden_act="silu",
               max_position_embeddings=40960, rms_norm_eps=1e-6, rope_theta=1000000, attention_bias=False,
               torch_dtype="bfloat16", bos_token_id=151643, eos_token_id=151645, **GEOMETRY[name])
    d = tempfile.mkdtemp(prefix=f"nvllm_{name}_")
    (Path(d) / "config.json").write_text(json.dumps(cfg))
    return d


def random_init(model, path=None, seed=0):
    """Stands in for nanovllm.utils.loader.load_model: same parameters, seeded random values."""
    import torch
    import torch.distributed as dist
    rank = dist.get_rank() if dist.is_initialized() else 0
    g = torch.Generator(device="cuda").manual_seed(1234 + seed + rank)
    with torch.no_grad():
        for pname, p in model.named_parameters():
            if "norm" in pname:
                p.fill_(1.0)
            else:
                p.normal_(0.0, 0.02, generator=g)


class _StubTokenizer:
    eos_token_id = -1

    def encode(self, text):
        return [1] * max(1, len(text))

    def decode(self, ids):
        return ""


def apply_shims(attn: str, ref_path: str):
    """Runs in every engine process (rank 0 and the spawned tensor-parallel workers)."""
    if ref_path not in sys.path:
        sys.path.insert(0, ref_path)
    if str(ROOT) not in sys.path:
        sys.path.insert(0, str(ROOT))
    if attn in ("b200", "b200-fused", "b200-full", "b200-full-ar", "b200-full-gemm-ar"):
        from nano_vllm_b200 import plugin
        plugin.install()
        if attn != "b200":
            plugin.fuse_pre_attention()
        if attn in ("b200-full", "b200-full-ar", "b200-full-gemm-ar"):
            plugin.fuse_sampler()
            plugin.fuse_decode_inputs()
        if attn in ("b200-full-ar", "b200-full-gemm-ar"):
            plugin.fuse_all_reduce(fuse_gemm=attn == "b200-full-gemm-ar")
            plugin.fuse_lm_head()
    import nanovllm.engine.model_runner as mr
    mr.load_model = random_init


def _worker(config_blob, rank, event, attn, ref_path):
    # The config travels as bytes: unpickling a nanovllm object would import the package (and
    # with it the stock attention module) before the swap below has been made.
    apply_shims(attn, ref_path)
    import pickle
    from nanovllm.engine.model_runner import ModelRunner
    ModelRunner(pickle.loads(config_blob), rank, event)


def make_engine(model_dir: str, attn: str, ref_path: str, **kwargs):
    """LLMEngine.__init__ (nanovllm/engine/llm_engine.py:17-34) with the shims applied in
    every process and the tokenizer stubbed; everything else is the reference's own object."""
    apply_shims(attn, ref_path)
    import torch.multiprocessing as mp
    from dataclasses import fields
    from nanovllm.config import Config
    from nanovllm.engine.llm_engine import LLMEngine
    from nanovllm.engine.model_runner import ModelRunner
    from nanovllm.engine.scheduler import Scheduler

    class Engine(LLMEngine):
        def __init__(self, model, **kw):
            names = {f.name for f in fields(Config)}
            config = Config(model, **{k: v for k, v in kw.items() if k in names})
            config.hf_config.rope_scaling = None
            self.ps, self.events = [], []
            ctx = mp.get_context("spawn")
            import pickle
            blob = pickle.dumps(config)
            for i in range(1, config.tensor_parallel_size):
                event = ctx.Event()
                proc = ctx.Process(target=_worker, args=(blob, i, event, attn, ref_path))
                proc.start()
                self.ps.append(proc)
                self.events.append(event)
            self.model_runner = ModelRunner(config, 0, self.events)
            self.tokenizer = _StubTokenizer()
            config.eos = self.tokenizer.eos_token_id
            self.scheduler = Scheduler(config)
            atexit.register(self.exit)

    return Engine(model_dir, **kwargs)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--attn", default="b200", choices=["b200", "b200-fused", "b200-full", "b200-full-ar", "b200-full-gemm-ar", "reference"],
                    help="b200: swap the attention layer; b200-fused: also fuse q/k norm + rotary + store; "
                         "b200-full: also the one-pass sampler and the one-launch decode inputs; b200-full-ar: also the "
                         "peer-memory all-reduce and the vocabulary-sharded sampling (TP > 1); b200-full-gemm-ar: also the "
                         "row-parallel projections and their sums as one launch; reference: stock nano-vllm")
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--model", default="qwen3-0.6b", choices=sorted(GEOMETRY))
    ap.add_argument("--num-seqs", type=int, default=256)
    ap.add_argument("--max-len", type=int, default=1024)
    ap.add_argument("--max-model-len", type=int, default=4096)
    ap.add_argument("--enforce-eager", action="store_true")
    ap.add_argument("--ref-path", default=str(ROOT / "baseline" / "_ref"))
    args = ap.parse_args()

    if not (Path(args.ref_path) / "nanovllm").is_dir():
        print(json.dumps({"unavailable": f"no nano-vllm install under {args.ref_path}"}))
        return
    try:  # a crashed earlier run can leave the engine's shared-memory segment behind
        os.unlink("/dev/shm/nanovllm")
    except OSError:
        pass
    os.chdir(tempfile.mkdtemp(prefix="nvllm_cwd_"))
    model_dir = write_model_dir(args.model)
    t0 = time.time()
    llm = make_engine(model_dir, args.attn, args.ref_path, enforce_eager=args.enforce_eager,
                      max_model_len=args.max_model_len, tensor_parallel_size=args.tp)
    init_s = time.time() - t0
    from nanovllm.sampling_params import SamplingParams

    random.seed(0)
    vocab = 151936
    prompts = [[random.randint(0, vocab - 1) for _ in range(random.randint(100, args.max_len))]
               for _ in range(args.num_seqs)]
    sps = [SamplingParams(temperature=0.6, ignore_eos=True, max_tokens=random.randint(100, args.max_len))
           for _ in range(args.num_seqs)]
    llm.generate([[1, 2, 3, 4, 5, 6, 7, 8]], SamplingParams(temperature=0.6, max_tokens=8, ignore_eos=True), use_tqdm=False)
    import torch
    torch.cuda.synchronize()
    t = time.time()
    outs = llm.generate(prompts, sps, use_tqdm=False)
    torch.cuda.synchronize()
    dt = time.time() - t
    total = sum(sp.max_tokens for sp in sps)
    got = sum(len(o["token_ids"]) for o in outs)
    line = {"metric": "e2e_output_tok_per_s", "value": round(total / dt, 1), "unit": "tok/s", "attn": args.attn,
            "model": args.model + " (random init)", "tp": args.tp, "num_seqs": args.num_seqs,
            "output_tokens": total, "tokens_returned": got, "prompt_tokens": sum(map(len, prompts)),
            "seconds": round(dt, 3), "engine_init_s": round(init_s, 1), "cuda_graphs": not args.enforce_eager}
    if args.attn != "reference":
        from nano_vllm_b200 import _lib
        line["kernel_launches"] = _lib.launch_count()
        line["device_status_word"] = _lib.read_status()
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
