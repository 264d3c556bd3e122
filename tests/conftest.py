import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tt-xla_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)

# Attention parity budget: bf16 outputs against the fp32 oracle.
MAX_ABS_TOL = 2e-2
MEAN_ABS_TOL = 2e-3


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def assert_attention_close(out: torch.Tensor, ref_fp32: torch.Tensor, what: str = "") -> None:
    """bf16 kernel output vs fp32 oracle: max |d| <= 2e-2 and mean |d| <= 2e-3."""
    d = (out.detach().float().cpu() - ref_fp32.detach().float().cpu()).abs()
    assert torch.isfinite(d).all(), f"{what}: non-finite values in the comparison"
    mx, mean = d.max().item(), d.mean().item()
    assert mx <= MAX_ABS_TOL and mean <= MEAN_ABS_TOL, (
        f"{what}: max abs {mx:.3e} (limit {MAX_ABS_TOL}), mean abs {mean:.3e} "
        f"(limit {MEAN_ABS_TOL})"
    )


@pytest.fixture(scope="session")
def built_library():
    """Builds (or reuses) libb200attn.so in-tree; returns its path."""
    from b200attn.build import build_library

    return build_library()


@pytest.fixture()
def clean_error_word():
    """Asserts that no kernel reported a device-side problem during the test."""
    from b200attn import ops

    ops.read_error_word()
    yield
    assert ops.read_error_word() == 0, "a kernel set the device diagnostics word"
