"""Decode-step inputs expanded on the GPU into a graph's static tensors, against the restated
reference semantics (clear, then copy the first rows; block tables padded with -1)."""
import random

import numpy as np
import pytest
import torch

import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent / "golden"))
import cases as C  # noqa: E402

from nano_vllm_b200 import _lib, decode_inputs as DI
from oracle import paged_attention_ref as R
from test_decode_inputs_host import make_seqs

pytestmark = pytest.mark.gpu

GRAPH_BS = [1, 2, 4, 8] + list(range(16, 513, 16))


def _graph_vars(cuda, rows, width, fill):
    return {"input_ids": torch.full((rows,), fill, dtype=torch.int64, device=cuda),
            "positions": torch.full((rows,), fill, dtype=torch.int64, device=cuda),
            "slot_mapping": torch.full((rows,), fill, dtype=torch.int32, device=cuda),
            "context_lens": torch.full((rows,), fill, dtype=torch.int32, device=cuda),
            "block_tables": torch.full((rows, width), fill, dtype=torch.int32, device=cuda)}


@pytest.mark.parametrize("width,max_len", [(16, 4096), (160, 40960)])
def test_steps_of_changing_batch_size(cuda, width, max_len):
    """A run of steps whose batch grows and shrinks: after each, the rows the graph of that size
    reads equal the reference's buffers bit for bit, rows beyond keep what they had."""
    rng = random.Random(width)
    gv = _graph_vars(cuda, 512, width, 7)
    stager = DI.DecodeInputStager(512, width, cuda)
    touched = 0
    for n in [300, 256, 17, 16, 1, 512, 3, 130]:
        seqs = make_seqs(rng, n, max_len=max_len)
        gbs = next(x for x in GRAPH_BS if x >= n)
        temps = stager.stage(seqs, gbs, gv)
        torch.cuda.synchronize()
        ref = R.decode_inputs_ref(seqs, gbs, width)
        for k, want in ref.items():
            got = gv[k][:gbs].cpu().numpy()
            assert got.dtype == want.dtype and np.array_equal(got, want), f"{k} differs at batch {n}"
        assert np.array_equal(temps.cpu().numpy(), np.array([s.temperature for s in seqs], np.float32))
        touched = max(touched, gbs)
        for k in gv:
            assert (gv[k][touched:] == 7).all(), f"{k}: rows beyond the graph's batch were written"
    assert _lib.read_status() == 0


def test_bad_arguments_are_refused(cuda, lib):
    gv = _graph_vars(cuda, 16, 16, 0)
    staged = torch.zeros(4096, dtype=torch.uint8, device=cuda)
    ptrs = [gv[k].data_ptr() for k in ("input_ids", "positions", "slot_mapping", "context_lens", "block_tables")]
    off = DI.layout(4)
    ok = (staged.data_ptr(), off["tokens"], off["lens"], off["offsets"], off["blocks"], 4, 8, 2, 16, *ptrs, 16, None)
    assert lib.nvllm_decode_step_inputs(*ok) == 0
    torch.cuda.synchronize()

    def call(**kw):
        names = ["staged", "tokens_off", "lens_off", "offsets_off", "blocks_off", "batch", "graph_batch", "used_width",
                 "table_width", "input_ids", "positions", "slot_mapping", "context_lens", "block_tables", "stride", "stream"]
        args = dict(zip(names, ok))
        args.update(kw)
        return lib.nvllm_decode_step_inputs(*[args[k] for k in names])

    assert call(staged=None) == -1 and call(block_tables=None) == -1
    assert call(batch=9) == -3 and call(used_width=17) == -3 and call(stride=8) == -3 and call(table_width=0) == -3
    assert call(tokens_off=4) == -2 and call(lens_off=2) == -2
    assert b"decode_step_inputs" in lib.nvllm_last_error()


@pytest.mark.parametrize("name", ["few", "graph_batch", "one", "ragged"])
def test_recorded_reference_batches(cuda, name):
    """Batches for which nano-vllm's own prepare_decode / prepare_sample output was recorded."""
    seqs, rec = C.decode_input_cases()[name]
    n, widest = len(seqs), rec["block_tables"].shape[1]
    gbs = next(x for x in GRAPH_BS if x >= n)
    gv = _graph_vars(cuda, 512, 16, 9)
    temps = DI.DecodeInputStager(512, 16, cuda).stage(seqs, gbs, gv)
    torch.cuda.synchronize()
    for k in ("input_ids", "positions", "slot_mapping", "context_lens"):
        got = gv[k][:gbs].cpu().numpy()
        assert np.array_equal(got[:n], rec[k]) and not got[n:].any(), k
    bt = gv["block_tables"][:gbs].cpu().numpy()
    assert np.array_equal(bt[:n, :widest], rec["block_tables"]) and not bt[:, widest:].any() and not bt[n:].any()
    assert np.array_equal(temps.cpu().numpy(), rec["temperatures"])
