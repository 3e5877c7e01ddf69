"""Records nano-vllm's own RMSNorm and RotaryEmbedding modules (nanovllm/layers/layernorm.py,
rotary_embedding.py) on seeded q/k heads, on the CPU, in the order its Qwen3 attention block
applies them (nanovllm/models/qwen3.py:89-105).

    TORCHDYNAMO_DISABLE=1 python tests/golden/make_pre_attention_golden.py /path/to/nano-vllm-checkout

Both modules decorate their forward with torch.compile; with dynamo disabled the same Python
bodies run eagerly, which needs no GPU and no compiler.
"""
import importlib.util
import os
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
CASES = {
    # name: (seed, tokens, q heads, kv heads, head_dim, with q/k norm, rope base, max position)
    "qwen3": (51, 37, 16, 8, 128, True, 1000000.0, 4096),
    "qwen3_8b_shard": (52, 9, 8, 2, 128, True, 1000000.0, 40960),
    "qwen2": (53, 21, 14, 2, 64, False, 1000000.0, 32768),
}


def load(ref_root, name):
    spec = importlib.util.spec_from_file_location("ref_" + name, ref_root / "nanovllm" / "layers" / (name + ".py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main():
    assert os.environ.get("TORCHDYNAMO_DISABLE") == "1", "run with TORCHDYNAMO_DISABLE=1"
    ref_root = Path(sys.argv[1])
    ln, rope = load(ref_root, "layernorm"), load(ref_root, "rotary_embedding")
    out = {}
    for name, (seed, n, hq, hkv, d, norm, base, max_pos) in CASES.items():
        g = torch.Generator().manual_seed(seed)
        qkv = (torch.randn(n, (hq + 2 * hkv) * d, generator=g) * 1.5).to(torch.bfloat16)
        positions = torch.randint(0, max_pos, (n,), generator=g)
        q, k, _ = qkv.split([hq * d, hkv * d, hkv * d], dim=-1)
        if norm:
            qn, kn = ln.RMSNorm(d, eps=1e-6).to(torch.bfloat16), ln.RMSNorm(d, eps=1e-6).to(torch.bfloat16)
            with torch.no_grad():
                qn.weight.copy_((1 + 0.1 * torch.randn(d, generator=g)).to(torch.bfloat16))
                kn.weight.copy_((1 + 0.1 * torch.randn(d, generator=g)).to(torch.bfloat16))
                q = qn(q.reshape(n, hq, d).clone()).reshape(n, hq * d)
                k = kn(k.reshape(n, hkv, d).clone()).reshape(n, hkv * d)
            out[f"{name}.q_weight"] = qn.weight.detach().view(torch.int16).numpy()
            out[f"{name}.k_weight"] = kn.weight.detach().view(torch.int16).numpy()
        rot = rope.RotaryEmbedding(d, d, max_pos, base)
        with torch.no_grad():
            q, k = rot(positions, q.contiguous(), k.contiguous())
        out[f"{name}.qkv"] = qkv.view(torch.int16).numpy()
        out[f"{name}.positions"] = positions.numpy()
        out[f"{name}.q"] = q.reshape(n, hq, d).contiguous().view(torch.int16).numpy()
        out[f"{name}.k"] = k.reshape(n, hkv, d).contiguous().view(torch.int16).numpy()
        out[f"{name}.geometry"] = np.array([hq, hkv, d, int(norm), max_pos], np.int64)
        out[f"{name}.rope_base"] = np.float64(base)
        rows = torch.tensor([0, 1, max_pos // 2, max_pos - 1])
        out[f"{name}.cache_rows"] = rot.cos_sin_cache[rows].numpy()
    np.savez_compressed(HERE / "pre_attention.npz", **out)
    print({k: v.shape for k, v in out.items() if k.startswith("qwen3.")})


if __name__ == "__main__":
    main()
