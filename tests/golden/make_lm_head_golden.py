"""Records nano-vllm's own ParallelLMHead + Sampler under emulated tensor parallelism, on the CPU.

    python tests/golden/make_lm_head_golden.py /path/to/nano-vllm-checkout

``torch.distributed`` is patched the way the reference's own examples/test_parallel_lmhead.py does
it: ``get_rank`` / ``get_world_size`` return the emulated rank and size while a head is built and
run, and ``gather`` hands rank 0 the logits the other ranks computed.  Each rank's module gets its
slice of one seeded [V, H] matrix through the module's own ``weight_loader``.  Stored: the seeded
inputs' seeds, the temperatures, and the tokens rank 0's Sampler returned (its exponential draw is
reproducible from the stored seed with one ``exponential_`` call on a [B, V] tensor).
"""
import sys
from pathlib import Path
from unittest.mock import patch

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
CASES = {
    # name: (seed, ranks, vocab, hidden, rows, sequence lengths for prefill or None, temperatures)
    "decode_tp1": (21, 1, 4096, 64, 5, None, [0.0, 0.6, 1.0, 0.0, 0.3]),
    "decode_tp2": (22, 2, 4096, 64, 5, None, [0.0, 0.6, 1.0, 0.0, 0.3]),
    "decode_tp4": (23, 4, 6000, 96, 6, None, [0.7, 0.0, 0.6, 2.0, 0.1, 0.0]),
    "decode_tp8": (24, 8, 151936, 32, 3, None, [0.6, 0.0, 1.0]),
    "prefill_tp2": (25, 2, 4096, 64, 11, [3, 1, 5, 2], [0.0, 0.6, 0.0, 1.2]),
    "prefill_tp4": (26, 4, 6000, 96, 9, [4, 5], [0.6, 0.0]),
}


def main():
    sys.path.insert(0, sys.argv[1])
    import torch.distributed as dist
    from nanovllm.layers.embed_head import ParallelLMHead
    from nanovllm.layers.sampler import Sampler
    from nanovllm.utils.context import reset_context, set_context

    out = {}
    for name, (seed, ranks, vocab, hidden, rows, lens, temps) in CASES.items():
        g = torch.Generator().manual_seed(seed)
        weight = torch.randn(vocab, hidden, generator=g).to(torch.bfloat16)
        x = torch.randn(rows, hidden, generator=g).to(torch.bfloat16)
        cu = None if lens is None else torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)
        partial = {}

        def fake_gather(tensor, gather_list, dst):
            if gather_list is not None:  # rank 0: the others have run before it
                for r in range(ranks):
                    gather_list[r].copy_(tensor if r == 0 else partial[r])

        logits = None
        for rank in list(range(1, ranks)) + [0]:
            with patch.object(dist, "get_rank", return_value=rank), patch.object(dist, "get_world_size", return_value=ranks), \
                    patch.object(dist, "gather", side_effect=fake_gather):
                head = ParallelLMHead(vocab, hidden).to(torch.bfloat16)
                head.weight.weight_loader(head.weight, weight)
                reset_context()
                if cu is None:
                    set_context(False)
                else:
                    set_context(True, cu_seqlens_q=cu)
                with torch.no_grad():
                    if ranks == 1:
                        logits = head(x)
                    elif rank == 0:
                        logits = head(x)
                    else:
                        # a worker rank's forward ends in the gather, which returns nothing to it;
                        # what it contributed is its local product
                        xs = x if cu is None else x[(cu[1:] - 1).to(torch.int64)].contiguous()
                        partial[rank] = torch.nn.functional.linear(xs, head.weight)
                        assert head(x) is None
                reset_context()
        t = torch.tensor(temps, dtype=torch.float32)
        torch.manual_seed(2000 + seed)
        tokens = Sampler()(logits.clone(), t)
        out[f"{name}.tokens"] = tokens.numpy()
        out[f"{name}.temperatures"] = t.numpy()
        out[f"{name}.seeds"] = np.array([seed, 2000 + seed], dtype=np.int64)
        out[f"{name}.shape"] = np.array([ranks, vocab, hidden, rows], dtype=np.int64)
        out[f"{name}.lens"] = np.array(lens if lens is not None else [], dtype=np.int64)
        if vocab <= 8192:
            out[f"{name}.logits"] = logits.view(torch.int16).numpy()
    np.savez_compressed(HERE / "lm_head.npz", **out)
    print({k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
