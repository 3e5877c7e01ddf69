"""Known-answer check of the tcgen05 / TMEM / TMA building blocks (nvllm_selftest_umma)."""
import pytest
import torch

from nano_vllm_b200 import _lib

pytestmark = pytest.mark.gpu


def test_umma_building_blocks_known_answer(cuda, lib):
    g = torch.Generator().manual_seed(71)
    a = torch.randn(128, 128, generator=g).bfloat16().to(cuda)
    b = torch.randn(128, 128, generator=g).bfloat16().to(cuda)
    out_ss = torch.full((128, 128), float("nan"), device=cuda)
    out_ts = torch.full((128, 128), float("nan"), device=cuda)
    _lib.check(lib.nvllm_selftest_umma(a.data_ptr(), b.data_ptr(), out_ss.data_ptr(), out_ts.data_ptr(),
                                       torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert _lib.read_status() == 0, "a bounded wait expired inside the self-test kernel"
    ref_ss = a.float() @ b.float().t()
    ref_ts = a.float() @ b.float()
    assert torch.allclose(out_ss, ref_ss, atol=1e-2, rtol=1e-3), (out_ss - ref_ss).abs().max()
    assert torch.allclose(out_ts, ref_ts, atol=1e-2, rtol=1e-3), (out_ts - ref_ts).abs().max()


def test_bounded_wait_expires_with_a_status_not_a_hang(cuda, lib):
    """Nothing signals the barrier: the wait must run out (~1 s), report NVLLM_STATUS_TIMEOUT and
    leave the context usable.  No fault is provoked."""
    import time
    _lib.read_status()
    res = torch.full((2,), -1, dtype=torch.int32, device=cuda)
    t0 = time.time()
    _lib.check(lib.nvllm_selftest_wait_expiry(res.data_ptr(), torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    dt = time.time() - t0
    assert res.tolist() == [0, 0]
    assert _lib.read_status() & 4
    assert 0.3 < dt < 10.0, dt
    # the context still works and the status word is clear again
    x = torch.ones(8, device=cuda)
    assert float(x.sum()) == 8.0 and _lib.read_status() == 0
