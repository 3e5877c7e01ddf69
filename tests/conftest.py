import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def lib():
    """The built C-ABI library (built on demand; nvcc cross-compiles without a GPU)."""
    from nano_vllm_b200 import _lib, build
    build.build()
    return _lib.load()


@pytest.fixture(scope="session")
def cuda(lib):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")


# max-abs / mean-abs bounds of bf16 attention outputs against the fp32 oracle
MAX_ABS_TOL = 2e-2
MEAN_ABS_TOL = 2e-3


def assert_close_to_oracle(out_bf16, ref_fp32, what=""):
    diff = (out_bf16.float().cpu() - ref_fp32).abs()
    assert not diff.isnan().any(), f"{what}: NaN in output"
    mx, mean = diff.max().item(), diff.mean().item()
    assert mx <= MAX_ABS_TOL and mean <= MEAN_ABS_TOL, f"{what}: max-abs {mx:.4g} mean-abs {mean:.4g}"
