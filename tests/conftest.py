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
def same_kernels_for_every_row_count():
    """One-token steps normally take their own decode-attention kernel, and calls of four rows and more may take the
    tensor-memory weight-streaming kernel; their rounding differs from the other kernels' by ~0.3 % of the logit scale, enough
    to flip a near-tie.  Bit-exact comparisons between one-row and many-row calls pin every row count to one kernel each."""
    from r4dx_b200 import native
    from r4dx_b200.ops import kernels as K
    impl = K.GEMV_IMPL
    native.cuda().r4dxb_set_attn_decode_row(0)
    K.set_gemv_impl("simt")
    yield
    K.set_gemv_impl(impl)
    native.cuda().r4dxb_set_attn_decode_row(1)
