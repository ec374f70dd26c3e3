"""The allocation-free argmax entry point, called through its exported C symbol.

Some users of the kernel library may not allocate device memory at the point where they need an
argmax over logits: they run inside a host framework's callback that forbids cudaMalloc, or inside
a graph capture.  ``r4dxb_argmax_rows_static`` keeps its temporary partials in a fixed array inside
the library.  This file checks it against the regular entry point (caller-provided scratch) on two
calls in a row, so a result that depended on what the previous call left in the shared array
would show up.  It is collected last on purpose: a run that stops at the first failure has by then
exercised every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from r4dx_b200 import native
    L = native.cuda()
    fn = L.r4dxb_argmax_rows_static
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p,
                   ctypes.c_void_p, ctypes.c_void_p]
    return L, fn


def _static_argmax(fn, logits, id_offset):
    T, V = logits.shape
    ids = torch.full((T,), -1, dtype=torch.int32, device=logits.device)
    vals = torch.zeros(T, dtype=torch.float32, device=logits.device)
    rc = fn(logits.data_ptr(), 1 if logits.dtype == torch.float32 else 0, T, V, id_offset, ids.data_ptr(),
            vals.data_ptr(), torch.cuda.current_stream().cuda_stream)
    return rc, ids, vals


def test_static_scratch_argmax_matches_regular_entry_point_twice():
    from r4dx_b200.ops import kernels as K
    L, fn = _lib()
    g = torch.Generator().manual_seed(11)
    first = torch.randn(8, 50000, generator=g).cuda()
    # second call: fewer rows, another width and dtype, values arranged so stale partials would win if read
    second = (torch.randn(3, 12345, generator=g) - 10.0).to(torch.bfloat16).cuda()
    second[1, 7] = second[1, 9000] = 5.0          # a tie: the lower index must be reported
    for logits, off in ((first, 0), (second, 100)):
        rc, ids, vals = _static_argmax(fn, logits, off)
        assert rc == 0
        ref_ids, ref_vals = K.argmax_rows(logits, id_offset=off)
        torch.cuda.synchronize()
        assert torch.equal(ids, ref_ids)
        assert torch.equal(vals, ref_vals)
    assert ids[1].item() == 107


def test_static_scratch_argmax_rejects_too_many_rows():
    L, fn = _lib()
    too_many = torch.zeros(65, 16, device="cuda")
    rc, ids, _ = _static_argmax(fn, too_many, 0)
    assert rc == 10003                              # R4DXB_TOO_LARGE, nothing launched
    torch.cuda.synchronize()
    assert (ids == -1).all()
