"""Row-parallel projection fused with its all-reduce (tcgen05 product, peer-memory epilogue), all
ranks emulated by one cooperative launch on one GPU, against the oracle's per-rank fp32 product
rounded to bf16 and summed in rank order."""
import pytest
import torch

from nano_vllm_b200 import _lib, allreduce as AR
from oracle import paged_attention_ref as R

pytestmark = pytest.mark.gpu
MAX_BYTES = 4 << 20


def _scratch(cuda, world):
    n = _lib.load().nvllm_ar_emulated_scratch_bytes(world, MAX_BYTES)
    return torch.zeros(n, dtype=torch.uint8, device=cuda)


def _small_ints(shape, g, density):
    """Values in {-1, 0, 1}: every product, partial sum and rounding below is exact in bf16 / fp32."""
    v = torch.randint(-1, 2, shape, generator=g).to(torch.float32)
    keep = torch.rand(shape, generator=g) < density
    return (v * keep).to(torch.bfloat16)


@pytest.mark.parametrize("mode", [1, 2])
@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("m,n,k", [(8, 256, 128), (200, 1024, 320), (128, 4096, 512), (1, 1024, 64), (40, 512, 6144),
                                   (256, 2048, 1536)])
def test_emulated_ranks_exact_on_integer_operands(cuda, world, m, n, k, mode):
    """Operands in {-1, 0, 1}: no rounding anywhere, so every rank must hold the oracle's bits, in
    one shot (every rank sums every tile; falls back to two where the cell areas are too small) and
    in two (the tile's owner sums).  Shapes: one ragged row tile; two row tiles with k not a multiple
    of the 64-element k-block; more tiles than thread blocks (a block loops); a single row; a small
    batch with a long k (short stages, the deep ring wraps); two full row tiles."""
    g = torch.Generator().manual_seed(1000 * world + m)
    xs = [_small_ints((m, k), g, 0.25) for _ in range(world)]
    ws = [_small_ints((n, k), g, 0.25) for _ in range(world)]
    want = R.row_parallel_linear_ref(xs, ws)
    assert want.abs().max() <= 256  # integers up to 256 are exact in bf16
    scratch = _scratch(cuda, world)
    for _ in range(3):  # the two cell areas alternate; the third call reuses the first
        outs = AR.linear_all_reduce_emulated([x.to(cuda) for x in xs], [w.to(cuda) for w in ws], scratch, MAX_BYTES, mode)
        torch.cuda.synchronize()
        for r, o in enumerate(outs):
            assert torch.equal(o.cpu().view(torch.int16), want.view(torch.int16)), f"rank {r}"
    assert _lib.read_status() == 0


@pytest.mark.parametrize("world", [2, 8])
def test_emulated_ranks_agree_and_match_oracle_on_random_operands(cuda, world):
    """Gaussian operands: the kernel's fp32 accumulation order differs from the oracle's, so a
    partial may round to the neighbouring bf16 value: tolerance = 2 bf16 steps of the largest
    output (2 x 2^-8 relative), and all ranks must hold the same bits."""
    m, n, k = 96, 1024, 512
    g = torch.Generator().manual_seed(world)
    xs = [torch.randn(m, k, generator=g).to(torch.bfloat16) for _ in range(world)]
    ws = [(torch.randn(n, k, generator=g) * k ** -0.5).to(torch.bfloat16) for _ in range(world)]
    want = R.row_parallel_linear_ref(xs, ws).to(torch.float32)
    outs = AR.linear_all_reduce_emulated([x.to(cuda) for x in xs], [w.to(cuda) for w in ws], _scratch(cuda, world), MAX_BYTES)
    torch.cuda.synchronize()
    got = [o.cpu() for o in outs]
    for o in got[1:]:
        assert torch.equal(o.view(torch.int16), got[0].view(torch.int16))
    tol = 2 * 2.0 ** -8 * float(want.abs().max())
    assert float((got[0].to(torch.float32) - want).abs().max()) <= tol
    assert _lib.read_status() == 0


def test_emulated_fused_and_plain_calls_share_the_cell_areas(cuda):
    """Fused projections and plain all-reduces of every cell protocol, interleaved on one area: the
    call counts and the two alternating cell areas are common to both."""
    world = 4
    scratch = _scratch(cuda, world)
    g = torch.Generator().manual_seed(7)
    for step in range(6):
        if step % 2 == 0:
            xs = [_small_ints((64, 256), g, 0.25) for _ in range(world)]
            ws = [_small_ints((512, 256), g, 0.25) for _ in range(world)]
            outs = AR.linear_all_reduce_emulated([x.to(cuda) for x in xs], [w.to(cuda) for w in ws], scratch, MAX_BYTES,
                                                 mode=1 + step // 2 % 2)
            want = R.row_parallel_linear_ref(xs, ws)
        else:
            xs = [(torch.randn(64 * 512, generator=g) * 2).to(torch.bfloat16) for _ in range(world)]
            outs = AR.all_reduce_emulated([x.to(cuda) for x in xs], scratch, MAX_BYTES, protocol=1 if step % 4 == 1 else 4)
            want = R.allreduce_ref(xs)
        torch.cuda.synchronize()
        for r, o in enumerate(outs):
            assert torch.equal(o.cpu().view(torch.int16), want.view(torch.int16)), f"step {step}, rank {r}"
    assert _lib.read_status() == 0


def test_shapes_the_kernel_refuses(cuda):
    lib = _lib.load()
    assert lib.nvllm_ar_gemm_tile(256, 4096, 512, 8, 8 << 20) == 64
    assert lib.nvllm_ar_gemm_tile(64, 4096, 512, 8, 8 << 20) == 32
    assert lib.nvllm_ar_gemm_tile(1024, 4096, 512, 8, 8 << 20) == 0   # cell areas too small
    assert lib.nvllm_ar_gemm_tile(8, 4096, 100, 2, 8 << 20) == 0      # k not a multiple of 8
    assert lib.nvllm_ar_gemm_tile(8, 48, 64, 2, 8 << 20) == 0         # n not a multiple of 32
    assert lib.nvllm_ar_gemm_tile(8, 64, 64, 4, 8 << 20) == 32        # fewer tiles than ranks: one shot
    x = torch.zeros(8, 64, dtype=torch.bfloat16, device=cuda)
    w = torch.zeros(48, 64, dtype=torch.bfloat16, device=cuda)
    with pytest.raises(RuntimeError):
        AR.linear_all_reduce_emulated([x, x], [w, w], _scratch(cuda, 2), MAX_BYTES)
