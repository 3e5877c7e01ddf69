"""One-pass token sampling on the GPU, through the C ABI: the reference Sampler's recorded
decisions for a given exponential draw, exact greedy rows, and the distribution of the
kernel's own Philox draws."""
import math
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

sys.path.insert(0, str(Path(__file__).resolve().parent / "golden"))
import cases as C  # noqa: E402

GOLDEN = C.GOLDEN_DIR

from nano_vllm_b200 import attention as A
from oracle import paged_attention_ref as R

pytestmark = pytest.mark.gpu


def _same_decision(tokens, ref_tokens, scores, rel=1e-4):
    """Equal, or the two candidates' scores tie to within ``rel`` (the kernel decides in the
    log domain, the reference on probability ratios; roundings may order a near-tie either way)."""
    for b, (t, r) in enumerate(zip(tokens.tolist(), ref_tokens.tolist())):
        if t != r:
            st, sr = float(scores[b, t]), float(scores[b, r])
            assert st >= sr * (1 - rel) - 1e-30, f"row {b}: token {t} (score {st}) instead of {r} (score {sr})"


@pytest.mark.parametrize("name", ["ragged_vocab", "small", "wide"])
def test_recorded_reference_decisions(cuda, name):
    logits, temperatures, noise, tokens = C.sampler_cases()[name]
    got = A.sample_tokens(logits.to(cuda), temperatures.to(cuda), noise=noise.to(cuda)).cpu()
    _same_decision(got, tokens, R.sampler_scores_ref(logits, temperatures, noise))
    assert (got == tokens).float().mean() >= 0.75


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("vocab,stride", [(151936, 151936), (1000, 1000), (1237, 1237), (1237, 1243), (7, 9), (1, 1)])
def test_greedy_rows_are_argmax(cuda, dtype, vocab, stride):
    """Temperature 0: exactly the first index of the row maximum, for aligned rows (16-byte
    loads), rows that start off a 16-byte boundary, and vocabularies that are no multiple of 8."""
    g = torch.Generator().manual_seed(vocab + stride)
    B = 9
    buf = torch.randn(B, stride, generator=g).to(dtype)
    buf[0, : min(vocab, 5)] = 4.0  # a tie at the maximum: the lowest index wins
    buf[0, 0] = 100.0 if vocab > 1 else buf[0, 0]
    buf[1, vocab - 1] = 50.0       # maximum in the last (tail) position
    logits = buf.to(cuda)[:, :vocab]
    got = A.sample_tokens(logits, torch.zeros(B, device=cuda)).cpu()
    assert torch.equal(got, buf[:, :vocab].float().argmax(-1))
    assert int(got[1]) == vocab - 1


def test_ties_go_to_the_lowest_index(cuda):
    logits = torch.zeros(3, 4096, dtype=torch.bfloat16, device=cuda)
    logits[1, 77] = 1.0
    logits[1, 3000] = 1.0
    logits[2] = float("-inf")
    got = A.sample_tokens(logits, torch.zeros(3, device=cuda)).tolist()
    assert got == [0, 77, 0]


def test_own_draws_are_reproducible_and_advance_with_step(cuda):
    g = torch.Generator().manual_seed(5)
    logits = torch.randn(64, 32000, generator=g).to(torch.bfloat16).to(cuda)
    t = torch.full((64,), 1.0, device=cuda)
    a = A.sample_tokens(logits, t, seed=123, step=1)
    b = A.sample_tokens(logits, t, seed=123, step=1)
    c = A.sample_tokens(logits, t, seed=123, step=2)
    d = A.sample_tokens(logits, t, seed=124, step=1)
    assert torch.equal(a, b)
    assert (a != c).float().mean() > 0.5 and (a != d).float().mean() > 0.5
    # rows with identical logits still draw independently
    same = logits[:1].expand(64, -1).contiguous()
    e = A.sample_tokens(same, t, seed=9, step=1)
    assert e.unique().numel() > 32


@pytest.mark.parametrize("vocab,temperature", [(50, 1.0), (50, 0.6), (1000, 1.5), (37, 0.25)])
def test_own_draws_follow_the_softmax_distribution(cuda, vocab, temperature):
    """Chi-square goodness of fit of 400 000 draws against softmax(logits / T), plus a direct
    check on the rarest tokens (their chance hangs on the smallest exponential draws)."""
    g = torch.Generator().manual_seed(vocab)
    row = torch.randn(vocab, generator=g) * 2.0
    n = 400_000
    logits = row.to(torch.bfloat16).to(cuda).unsqueeze(0).expand(n, -1).contiguous()
    t = torch.full((n,), temperature, device=cuda)
    tokens = A.sample_tokens(logits, t, seed=2024, step=7)
    counts = torch.bincount(tokens, minlength=vocab).double().cpu()
    p = torch.softmax(row.to(torch.bfloat16).double() / temperature, dim=-1)
    expected = p * n
    keep = expected >= 10  # chi-square needs populated cells; pool the rest into one
    chi = float((((counts - expected) ** 2) / expected)[keep].sum())
    dof = int(keep.sum()) - 1
    if (~keep).any():
        e_rest, c_rest = float(expected[~keep].sum()), float(counts[~keep].sum())
        if e_rest >= 10:
            chi += (c_rest - e_rest) ** 2 / e_rest
            dof += 1
    # mean dof, variance 2*dof: six sigma above the mean practically never happens by chance
    assert chi < dof + 6 * math.sqrt(2 * dof), f"chi2 {chi:.1f} for {dof} degrees of freedom"
    rare = (expected >= 20) & (p < 2e-3)
    if rare.any():
        ratio = float(counts[rare].sum() / expected[rare].sum())
        assert abs(ratio - 1) < 6 / math.sqrt(float(expected[rare].sum())), f"rare tokens drawn {ratio:.3f}x as often as expected"


def test_mixed_temperatures_in_one_batch(cuda):
    g = torch.Generator().manual_seed(8)
    logits = (torch.randn(16, 151936, generator=g) * 2).to(torch.bfloat16)
    t = torch.tensor([0.0, 0.6] * 8)
    got = A.sample_tokens(logits.to(cuda), t.to(cuda), seed=1, step=1).cpu()
    assert torch.equal(got[0::2], logits.float().argmax(-1)[0::2])
    assert (got[1::2] != logits.float().argmax(-1)[1::2]).any()
    assert int(got.min()) >= 0 and int(got.max()) < 151936


def test_bad_arguments_are_refused(cuda, lib):
    logits = torch.zeros(2, 16, dtype=torch.bfloat16, device=cuda)
    t = torch.zeros(2, device=cuda)
    out = torch.zeros(2, dtype=torch.int64, device=cuda)
    assert lib.nvllm_sample_tokens(None, 0, 16, t.data_ptr(), None, 0, 0, 0, out.data_ptr(), 2, 16, None) == -1
    assert lib.nvllm_sample_tokens(logits.data_ptr(), 0, 8, t.data_ptr(), None, 0, 0, 0, out.data_ptr(), 2, 16, None) == -3
    assert lib.nvllm_sample_tokens(logits.data_ptr(), 0, 16, t.data_ptr(), None, 0, 0, 0, out.data_ptr(), 2, 0, None) == -3
    assert lib.nvllm_sample_tokens(logits.data_ptr(), 0, 16, t.data_ptr(), None, 0, 0, 0, out.data_ptr(), 0, 16, None) == 0
    assert b"sample_tokens" in lib.nvllm_last_error()
    with pytest.raises(AssertionError):
        A.sample_tokens(logits.half(), t)


# ---- vocabulary-sharded sampling (tensor-parallel LM head tail) ---------------------------------

def _merge(cands):
    """What dist.reduce(op=MAX) does over the ranks' candidate tensors."""
    best = cands[0]
    for c in cands[1:]:
        best = torch.maximum(best, c)
    return best


def test_sharded_candidates_reproduce_the_reference_lm_head_and_sampler(cuda):
    """nano-vllm's own ParallelLMHead + Sampler under 1, 2, 4, 8 emulated ranks
    (tests/golden/lm_head.npz): every rank's slice of the logits goes through
    nvllm_sample_candidates with the slice of the recorded draw, the candidates are merged by a
    MAX, and the unpacked tokens must be the reference's (or tie with them to 1e-4 relative)."""
    import sys
    from pathlib import Path
    sys.path.insert(0, str(Path(__file__).resolve().parent))
    from test_oracle_golden import _lm_head_case
    z = np.load(GOLDEN / "lm_head.npz")
    for name in sorted({k.split(".")[0] for k in z.files}):
        ranks, weight, x, cu, temps, noise = _lm_head_case(z, name)
        want, logits = R.lm_head_sample_ref(x, list(weight.chunk(ranks, 0)), cu, temps, noise)
        assert want.tolist() == z[f"{name}.tokens"].tolist()
        per = logits.shape[1] // ranks
        cands = []
        for r in range(ranks):
            sl = slice(r * per, (r + 1) * per)
            cands.append(A.sample_candidates(logits[:, sl].contiguous().to(cuda), temps.to(cuda), r * per,
                                             noise=noise[:, sl].contiguous().to(cuda)))
        got = A.sample_unpack(_merge(cands)).cpu()
        scores = R.sampler_scores_ref(logits, temps, noise)
        for b in range(temps.numel()):
            t, w = int(got[b]), int(want[b])
            assert t == w or float(scores[b, t]) >= float(scores[b, w]) * (1 - 1e-4), f"{name} row {b}: {t} vs {w}"


@pytest.mark.parametrize("ranks,vocab", [(2, 4096), (4, 6000), (8, 151936), (3, 1236), (2, 1002)])
def test_sharded_candidates_pick_the_token_of_the_one_rank_kernel(cuda, ranks, vocab):
    """Generated noise depends on (seed, step, row, global position) only, so slicing the
    vocabulary must not change a single token: aligned slices, slices that do not start on a
    group of four positions, greedy and sampled rows."""
    g = torch.Generator().manual_seed(vocab + ranks)
    logits = (torch.randn(7, vocab, generator=g) * 3).to(torch.bfloat16).to(cuda)
    temps = torch.tensor([0.0, 0.6, 1.0, 0.0, 2.0, 0.3, 0.6], device=cuda)
    per = vocab // ranks
    for step in (1, 2, 99):
        whole = A.sample_tokens(logits, temps, seed=5, step=step)
        cands = [A.sample_candidates(logits[:, r * per:(r + 1) * per].contiguous(), temps, r * per, seed=5, step=step)
                 for r in range(ranks)]
        assert torch.equal(A.sample_unpack(_merge(cands)), whole)
    # a slice with nothing to offer (all NaN) loses against any real candidate
    nan_slice = torch.full((7, per), float("nan"), dtype=torch.bfloat16, device=cuda)
    real = logits[:, :per].contiguous()
    merged = _merge([A.sample_candidates(real, temps, 0, seed=5, step=1), A.sample_candidates(nan_slice, temps, per, seed=5, step=1)])
    assert torch.equal(A.sample_unpack(merged), A.sample_tokens(real, temps, seed=5, step=1))
