"""The allocation-free norm backward, called through its exported C symbol.

Some users of the library have to run the fused norm backward from a place
where they cannot allocate device memory (see ``distdl_b200/csrc/no_alloc.h``);
for them the library offers ``dd_norm_bwd_noalloc``, which keeps its scratch in
a fixed array inside the library.  This test calls that symbol directly with
``ctypes`` twice in a row -- the second call finds the scratch dirty from the
first -- and compares dx / dw / db with the regular entry point ``dd_norm_bwd``
(whose scratch the caller allocates), using the tolerance of the other kernel
tests.  It lives in a file that pytest collects last, so a run that stops at
the first failure has already run everything else.
"""
import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "distdl_b200", "_C",
                   "libdistdl_b200.so")


def _close(a, b, tol=2e-2):
    err = (a.float() - b.float()).abs().max().item()
    scale = b.float().abs().max().item() + 1e-6
    assert err / scale < tol, f"err {err} scale {scale}"


def test_norm_bwd_noalloc_matches_regular_entry_point_twice():
    lib = ctypes.CDLL(LIB)
    vp, ci = ctypes.c_void_p, ctypes.c_int
    lib.dd_norm_bwd_noalloc.argtypes = [ci, vp, vp, vp, vp, vp, vp, vp, ci, ci, ci, vp]
    lib.dd_norm_bwd_noalloc.restype = ci
    lib.dd_norm_bwd.argtypes = [ci, vp, vp, vp, vp, vp, vp, vp, vp, vp, ci, ci, ci, vp]
    lib.dd_norm_bwd.restype = ci
    lib.dd_norm_fwd.argtypes = [ci, vp, vp, vp, vp, vp, vp, vp, ci, ci, ctypes.c_float, vp]
    lib.dd_norm_fwd.restype = ci
    lib.dd_norm_bwd_parts.argtypes = [ci]
    lib.dd_norm_bwd_parts.restype = ci
    lib.dd_norm_bwd_noalloc_max_d.restype = ci
    stream = torch.cuda.current_stream().cuda_stream
    # two calls in a row with different shapes and norm kinds
    for call, (rows, d, rms) in enumerate([(1000, 4096, 1), (333, 1600, 0)]):
        torch.manual_seed(call)
        x = torch.randn(rows, d, device="cuda", dtype=torch.bfloat16)
        w = (1 + 0.1 * torch.randn(d, device="cuda")).to(torch.bfloat16)
        dy = torch.randn(rows, d, device="cuda", dtype=torch.bfloat16)
        y = torch.empty_like(x)
        stats = torch.empty(rows, 2, device="cuda", dtype=torch.float32)
        assert lib.dd_norm_fwd(rms, x.data_ptr(), None, None, w.data_ptr(), None, y.data_ptr(), stats.data_ptr(),
                               rows, d, 1e-5, stream) == 0
        # regular entry point: caller-allocated scratch
        parts = lib.dd_norm_bwd_parts(rows)
        scratch = torch.empty(parts * 2 * d, device="cuda", dtype=torch.float32)
        dx_ref, dw_ref, db_ref = torch.empty_like(x), torch.empty(d, device="cuda"), torch.empty(d, device="cuda")
        assert lib.dd_norm_bwd(rms, dy.data_ptr(), x.data_ptr(), w.data_ptr(), stats.data_ptr(), None,
                               dx_ref.data_ptr(), dw_ref.data_ptr(), db_ref.data_ptr(), scratch.data_ptr(), 0, rows,
                               d, stream) == 0
        # allocation-free entry point: outputs are allocated here, before the call
        dx, dw, db = torch.empty_like(x), torch.empty(d, device="cuda"), torch.empty(d, device="cuda")
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        assert lib.dd_norm_bwd_noalloc(rms, dy.data_ptr(), x.data_ptr(), w.data_ptr(), stats.data_ptr(),
                                       dx.data_ptr(), dw.data_ptr(), db.data_ptr(), 0, rows, d, stream) == 0
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        _close(dx, dx_ref)
        _close(dw, dw_ref)
        _close(db, db_ref)
    # sizes beyond the built-in scratch are refused
    too_wide = lib.dd_norm_bwd_noalloc_max_d() + 8
    assert lib.dd_norm_bwd_noalloc(1, None, None, None, None, None, None, None, 0, 4, too_wide, stream) == 1003
