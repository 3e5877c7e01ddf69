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
