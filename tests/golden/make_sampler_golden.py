"""Records nano-vllm's own Sampler (nanovllm/layers/sampler.py) on seeded inputs, on the CPU.

    python tests/golden/make_sampler_golden.py /path/to/nano-vllm-checkout

The sampler is plain torch, so it runs without a GPU.  It draws its noise with a single
``exponential_`` call on a tensor shaped like the logits; re-seeding the generator and making
the same call yields the very draw it used, which is stored beside the tokens so that the
oracle and the CUDA kernel can be asked for the same decision.
"""
import importlib.util
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
CASES = {
    # name: (seed, batch, vocab, temperatures)
    "small": (11, 6, 1000, [0.0, 0.6, 1.0, 0.3, 0.0, 1.5]),
    "ragged_vocab": (12, 5, 1237, [0.7, 0.0, 0.6, 2.0, 0.1]),
    "wide": (13, 4, 151936, [0.6, 0.0, 1.0, 0.6]),
}


def main():
    ref_root = Path(sys.argv[1])
    spec = importlib.util.spec_from_file_location("ref_sampler", ref_root / "nanovllm" / "layers" / "sampler.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    sampler = mod.Sampler()
    out = {}
    for name, (seed, batch, vocab, temps) in CASES.items():
        g = torch.Generator().manual_seed(seed)
        logits = (torch.randn(batch, vocab, generator=g) * 3.0).to(torch.bfloat16)
        t = torch.tensor(temps, dtype=torch.float32)
        torch.manual_seed(1000 + seed)
        tokens = sampler(logits.clone(), t)
        torch.manual_seed(1000 + seed)
        noise = torch.empty(batch, vocab, dtype=torch.float32).exponential_(1)
        out[f"{name}.logits"] = logits.view(torch.int16).numpy()
        out[f"{name}.temperatures"] = t.numpy()
        # keep the file small: the noise of the wide case is regenerated from its seed by the tests
        if vocab <= 4096:
            out[f"{name}.noise"] = noise.numpy()
        else:
            del out[f"{name}.logits"]
        out[f"{name}.noise_seed"] = np.int64(1000 + seed)
        out[f"{name}.logits_seed"] = np.int64(seed)
        out[f"{name}.tokens"] = tokens.numpy()
    np.savez_compressed(HERE / "sampler.npz", **out)
    print({k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
