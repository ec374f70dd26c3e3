import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture
def same_attention_kernel_for_every_row_count():
    """One-token steps normally take their own decode-attention kernel, whose rounding differs from the window kernel's
    by ~0.3 % of the logit scale: enough to flip a near-tie.  Bit-exact comparisons between one-row and many-row calls
    pin both to the window kernel."""
    from r4dx_b200 import native
    native.cuda().r4dxb_set_attn_decode_row(0)
    yield
    native.cuda().r4dxb_set_attn_decode_row(1)
