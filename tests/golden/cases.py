"""Seeded cases shared by the golden-vector recorder (make_golden.py, runs the reference on a
GPU) and the tests that replay them (CPU oracle and CUDA kernels)."""
from __future__ import annotations

import hashlib
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[2]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from nano_vllm_b200 import workloads as W  # noqa: E402

GOLDEN_DIR = Path(__file__).resolve().parent


def decode_cases():
    return {
        "decode_qwen3_g2_d128": W.make_decode_case(101, 6, 1, 1, 16, 8, 128, context_lens=[1, 255, 256, 257, 1024, 700]),
        "decode_qwen3_8b_g4_d128": W.make_decode_case(102, 4, 1, 1, 8, 2, 128, context_lens=[100, 513, 2048, 1]),
        "decode_qwen2_g7_d64": W.make_decode_case(103, 5, 1, 1, 14, 2, 64, context_lens=[1, 255, 256, 257, 1024]),
    }


def prefill_cases():
    return {
        "prefill_packed_d128": W.make_prefill_case(201, 5, 1, 1, 4, 2, 128, share_every=0, lengths=[1, 100, 256, 257, 300]),
        "prefill_prefix_d128": W.make_prefill_case(202, 4, 1, 1, 4, 2, 128, lengths=[600, 600, 800, 1024],
                                                   shared_blocks=[0, 2, 0, 3]),
        "prefill_prefix_d64_g7": W.make_prefill_case(203, 3, 1, 1, 14, 2, 64, lengths=[300, 520, 257],
                                                     shared_blocks=[0, 1, 1]),
    }


def store_cases():
    """(key, value, k_cache, v_cache, slot_mapping) with permuted slots and a strided value."""
    out = {}
    for name, (seed, n, hkv, d) in {"store_qwen3": (301, 300, 8, 128), "store_qwen2": (302, 77, 2, 64)}.items():
        g = torch.Generator().manual_seed(seed)
        kv = torch.randn(n, 2 * hkv * d, generator=g).bfloat16()
        key, value = (t.view(n, hkv, d) for t in kv.split(hkv * d, dim=-1))  # both strided views
        k_cache = torch.randn(3, 256, hkv, d, generator=g).bfloat16()
        v_cache = torch.randn(3, 256, hkv, d, generator=g).bfloat16()
        slots = torch.randperm(3 * 256, generator=g)[:n].to(torch.int32)
        out[name] = (key, value, k_cache, v_cache, slots)
    return out


def sha(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def input_fingerprint(*tensors) -> str:
    """Detects a change in the seeded generators between recording and replay."""
    h = hashlib.sha256()
    for t in tensors:
        if t is not None:
            h.update(t.contiguous().view(torch.uint8).numpy().tobytes())
    return h.hexdigest()


# ---- sampler -------------------------------------------------------------------------------

def sampler_cases():
    """name -> (logits bf16 [B,V], temperatures fp32 [B], noise fp32 [B,V], tokens int64 [B]) as
    recorded by make_sampler_golden.py from nano-vllm's own Sampler on the CPU.  The widest
    case stores only its seeds; its logits and noise are drawn again here the way the
    recording script drew them."""
    from pathlib import Path
    import numpy as np
    z = np.load(Path(__file__).resolve().parent / "sampler.npz")
    names = sorted({k.split(".")[0] for k in z.files})
    out = {}
    for name in names:
        t = torch.from_numpy(z[f"{name}.temperatures"].copy())
        tokens = torch.from_numpy(z[f"{name}.tokens"].copy())
        batch = t.numel()
        if f"{name}.logits" in z.files:
            logits = torch.from_numpy(z[f"{name}.logits"].copy()).view(torch.bfloat16)
            noise = torch.from_numpy(z[f"{name}.noise"].copy())
        else:
            vocab = 151936
            g = torch.Generator().manual_seed(int(z[f"{name}.logits_seed"]))
            logits = (torch.randn(batch, vocab, generator=g) * 3.0).to(torch.bfloat16)
            state = torch.random.get_rng_state()
            torch.manual_seed(int(z[f"{name}.noise_seed"]))
            noise = torch.empty(batch, vocab, dtype=torch.float32).exponential_(1)
            torch.random.set_rng_state(state)
        out[name] = (logits, t, noise, tokens)
    return out


# ---- decode-step inputs ------------------------------------------------------------------------

class DecodeSeq:
    """The attributes of a nano-vllm Sequence that a decode step reads."""

    def __init__(self, last_token, num_tokens, temperature, block_table):
        self.last_token, self.num_tokens, self.temperature, self.block_table = last_token, num_tokens, temperature, block_table


def decode_input_cases():
    """name -> (sequences, recorded) where ``recorded`` holds what nano-vllm's own
    prepare_decode / prepare_block_tables / prepare_sample returned for them
    (make_decode_inputs_golden.py)."""
    import numpy as np
    z = np.load(GOLDEN_DIR / "decode_inputs.npz")
    out = {}
    for name in sorted({k.split(".")[0] for k in z.files}):
        lens = z[f"{name}.table_len"]
        ends = np.cumsum(lens)
        flat = z[f"{name}.table_flat"]
        seqs = [DecodeSeq(int(z[f"{name}.last_token"][i]), int(z[f"{name}.num_tokens"][i]), float(z[f"{name}.temperatures"][i]),
                          [int(b) for b in flat[ends[i] - lens[i]:ends[i]]]) for i in range(len(lens))]
        rec = {k: z[f"{name}.{k}"] for k in ("input_ids", "positions", "slot_mapping", "context_lens", "block_tables", "temperatures")}
        out[name] = (seqs, rec)
    return out


# ---- pre-attention step ------------------------------------------------------------------------

def pre_attention_cases():
    """name -> dict of what make_pre_attention_golden.py recorded from nano-vllm's own RMSNorm and
    RotaryEmbedding modules: inputs (qkv, positions, norm weights or None), geometry, outputs."""
    import numpy as np
    z = np.load(GOLDEN_DIR / "pre_attention.npz")
    bf16 = lambda a: torch.from_numpy(a.copy()).view(torch.bfloat16)
    out = {}
    for name in sorted({k.split(".")[0] for k in z.files}):
        hq, hkv, d, norm, max_pos = (int(v) for v in z[f"{name}.geometry"])
        out[name] = dict(hq=hq, hkv=hkv, d=d, max_pos=max_pos, base=float(z[f"{name}.rope_base"]),
                         qkv=bf16(z[f"{name}.qkv"]), positions=torch.from_numpy(z[f"{name}.positions"].copy()),
                         q_weight=bf16(z[f"{name}.q_weight"]) if norm else None,
                         k_weight=bf16(z[f"{name}.k_weight"]) if norm else None,
                         q=bf16(z[f"{name}.q"]), k=bf16(z[f"{name}.k"]),
                         cache_rows=torch.from_numpy(z[f"{name}.cache_rows"].copy()))
    return out
