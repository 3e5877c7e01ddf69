"""Host side of the one-copy decode-step inputs: the staging block against the restated
reference semantics, on the CPU."""
import random
from dataclasses import dataclass, field

import numpy as np
import pytest

from nano_vllm_b200 import decode_inputs as DI
from oracle import paged_attention_ref as R


@dataclass
class FakeSeq:
    """The attributes of nanovllm/engine/sequence.py's Sequence that a decode step reads."""
    last_token: int
    num_tokens: int
    temperature: float
    block_table: list = field(default_factory=list)


def make_seqs(rng, n, max_len=4096, num_blocks=5000):
    seqs = []
    for _ in range(n):
        length = rng.choice([1, 255, 256, 257, 512, 513, max_len]) if rng.random() < 0.3 else rng.randint(1, max_len)
        nblk = (length + 255) // 256
        seqs.append(FakeSeq(rng.randrange(151936), length, rng.choice([0.0, 0.6, 1.0]),
                            [rng.randrange(num_blocks) for _ in range(nblk)]))
    return seqs


@pytest.mark.parametrize("n", [1, 2, 7, 256, 512])
def test_staging_block_holds_the_step(n):
    rng = random.Random(n)
    seqs = make_seqs(rng, n)
    buf = np.full(DI.staging_bytes(512, 16), 0xAB, np.uint8)
    end, widest = DI.pack(seqs, buf)
    off = DI.layout(n)
    assert widest == max(len(s.block_table) for s in seqs)
    assert end == off["blocks"] + 4 * sum(len(s.block_table) for s in seqs)
    tokens = buf[off["tokens"]:off["lens"]].view(np.int64)
    lens = buf[off["lens"]:off["temperatures"]].view(np.int32)
    temps = buf[off["temperatures"]:off["offsets"]].view(np.float32)
    offs = buf[off["offsets"]:off["blocks"]].view(np.int32)
    blocks = buf[off["blocks"]:end].view(np.int32)
    ref = R.decode_inputs_ref(seqs, n, 16)
    assert np.array_equal(tokens, ref["input_ids"]) and np.array_equal(lens, ref["context_lens"])
    assert np.array_equal(temps, np.array([s.temperature for s in seqs], np.float32))
    for i, s in enumerate(seqs):
        assert list(blocks[offs[i]:offs[i + 1]]) == s.block_table
        assert list(ref["block_tables"][i, :len(s.block_table)]) == s.block_table
    assert (buf[end:] == 0xAB).all()  # nothing written past the step


def test_staging_block_too_small_is_refused():
    seqs = make_seqs(random.Random(0), 8)
    with pytest.raises(ValueError, match="too small"):
        DI.pack(seqs, np.zeros(64, np.uint8))


def test_sections_are_aligned_for_any_batch():
    for n in range(1, 600):
        off = DI.layout(n)
        assert off["tokens"] % 8 == 0 and all(off[k] % 4 == 0 for k in off)
        assert off["lens"] - off["tokens"] == 8 * n and off["blocks"] - off["offsets"] == 4 * (n + 1)


def test_worker_ranks_pack_sequences_without_sampling_parameters():
    """Sequences unpickled on a tensor-parallel worker have no ``temperature`` attribute."""
    class WorkerSeq:
        def __init__(self, s):
            self.last_token, self.num_tokens, self.block_table = s.last_token, s.num_tokens, s.block_table

    seqs = make_seqs(random.Random(3), 9)
    a = np.zeros(DI.staging_bytes(16, 16), np.uint8)
    b = np.zeros_like(a)
    end_a, _ = DI.pack(seqs, a)
    end_b, _ = DI.pack([WorkerSeq(s) for s in seqs], b, with_temperatures=False)
    off = DI.layout(9)
    assert end_a == end_b
    a[off["temperatures"]:off["offsets"]] = 0
    assert np.array_equal(a, b)
    with pytest.raises(AttributeError):
        DI.pack([WorkerSeq(s) for s in seqs], b)
