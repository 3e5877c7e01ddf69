"""Records what nano-vllm's own ModelRunner.prepare_decode / prepare_block_tables produce for
seeded batches of real Sequence objects, on the CPU.

    python tests/golden/make_decode_inputs_golden.py /path/to/nano-vllm-checkout

The two methods are called unbound on a stand-in runner that only has ``block_size``; the only
change made to them is that ``torch.tensor(..., pin_memory=True).cuda(non_blocking=True)`` stays
on the host (pinning and the copy need a GPU): inside the reference module ``torch.tensor`` drops
``pin_memory`` and ``Tensor.cuda`` returns the tensor itself while the methods run.  The context
they set is read back with the reference's own ``get_context``.
"""
import random
import sys
from pathlib import Path
from types import SimpleNamespace
from unittest import mock

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
CASES = {"one": (41, 1), "few": (42, 7), "graph_batch": (43, 256), "ragged": (44, 100)}


def make_sequences(Sequence, SamplingParams, seed, n):
    """Sequences in their decode phase: a prompt, a few generated tokens, a block table."""
    rng = random.Random(seed)
    seqs = []
    for _ in range(n):
        prompt = rng.choice([1, 255, 256, 257, 511, 512, 513]) if rng.random() < 0.4 else rng.randint(1, 3000)
        s = Sequence([rng.randrange(151936) for _ in range(prompt)], SamplingParams(temperature=rng.choice([0.0, 0.6, 1.0])))
        for _ in range(rng.randint(1, 300)):
            s.append_token(rng.randrange(151936))
        s.block_table = [rng.randrange(60000) for _ in range(s.num_blocks)]
        seqs.append(s)
    return seqs


def main():
    sys.path.insert(0, sys.argv[1])
    from nanovllm.engine import model_runner as mr
    from nanovllm.engine.sequence import Sequence
    from nanovllm.sampling_params import SamplingParams
    from nanovllm.utils.context import get_context, reset_context

    real_tensor = torch.tensor
    host_tensor = lambda data, **kw: real_tensor(data, **{k: v for k, v in kw.items() if k != "pin_memory"})
    runner = SimpleNamespace(block_size=256)
    runner.prepare_block_tables = lambda seqs: mr.ModelRunner.prepare_block_tables(runner, seqs)
    out = {}
    for name, (seed, n) in CASES.items():
        seqs = make_sequences(Sequence, SamplingParams, seed, n)
        with mock.patch.object(mr.torch, "tensor", host_tensor), \
                mock.patch.object(torch.Tensor, "cuda", lambda self, *a, **k: self):
            input_ids, positions = mr.ModelRunner.prepare_decode(runner, seqs)
            temperatures = mr.ModelRunner.prepare_sample(runner, seqs)
        ctx = get_context()
        assert not ctx.is_prefill
        out[f"{name}.input_ids"] = input_ids.numpy()
        out[f"{name}.positions"] = positions.numpy()
        out[f"{name}.slot_mapping"] = ctx.slot_mapping.numpy()
        out[f"{name}.context_lens"] = ctx.context_lens.numpy()
        out[f"{name}.block_tables"] = ctx.block_tables.numpy()
        out[f"{name}.temperatures"] = temperatures.numpy()
        # what the tests rebuild the sequences from
        out[f"{name}.last_token"] = np.array([s.last_token for s in seqs], np.int64)
        out[f"{name}.num_tokens"] = np.array([s.num_tokens for s in seqs], np.int32)
        out[f"{name}.table_flat"] = np.array([b for s in seqs for b in s.block_table], np.int32)
        out[f"{name}.table_len"] = np.array([len(s.block_table) for s in seqs], np.int32)
        reset_context()
    np.savez_compressed(HERE / "decode_inputs.npz", **out)
    print({k: v.shape for k, v in out.items() if k.startswith("ragged")})


if __name__ == "__main__":
    main()
