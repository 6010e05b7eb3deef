"""The allocation-free norm backward, called through its exported C symbol.

Some users of the library have to run the fused norm backward from a place
where they cannot allocate device memory (see ``distdl_b200/csrc/no_alloc.h``);
for them the library offers ``dd_norm_bwd_noalloc``, which keeps its scratch in
a fixed array inside the library.  This test calls that symbol directly with
``ctypes`` several times in a row -- every call after the first finds the
scratch dirty from the one before, and a small call follows a large one -- and
compares dx / dw / db with the regular entry point ``dd_norm_bwd`` (whose
scratch the caller allocates) and with an fp32 PyTorch restatement of the
operator.  Whether the call allocates is read from the driver's count of free
device memory, which also sees allocations made outside PyTorch.  It lives in a
file that pytest collects last, so a run that stops at the first failure has
already run everything else.
"""
import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "distdl_b200", "_C",
                   "libdistdl_b200.so")


def _close(a, b, tol):
    err = (a.float() - b.float()).abs().max().item()
    scale = b.float().abs().max().item() + 1e-6
    assert err / scale < tol, f"err {err} scale {scale}"


def _lib():
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
    return lib


def _torch_reference(rms, x, w, dy, eps=1e-5):
    """dx, dw, db of the norm in fp32 autograd."""
    xf = x.float().requires_grad_(True)
    wf = w.float().requires_grad_(True)
    bf = torch.zeros_like(wf, requires_grad=True)
    if rms:
        y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * wf + bf
    else:
        y = torch.nn.functional.layer_norm(xf, (x.shape[-1],), wf, bf, eps)
    y.backward(dy.float())
    return xf.grad, wf.grad, bf.grad


# (rows, d, rms, want dw/db, accumulate): a large call first, then small ones that
# use fewer scratch slices than the call before them left behind
CASES = [(1000, 4096, 1, True, 0), (333, 1600, 0, True, 0), (5, 4096, 1, True, 0), (700, 8192, 0, True, 1),
         (64, 1024, 1, False, 0), (3, 8192, 0, True, 1)]


def test_norm_bwd_noalloc_matches_regular_entry_point_on_calls_in_a_row():
    lib = _lib()
    stream = torch.cuda.current_stream().cuda_stream
    for call, (rows, d, rms, want_w, accumulate) in enumerate(CASES):
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
        start_w, start_b = torch.randn(d, device="cuda"), torch.randn(d, device="cuda")
        dx_ref, dw_ref, db_ref = torch.empty_like(x), start_w.clone(), start_b.clone()
        assert lib.dd_norm_bwd(rms, dy.data_ptr(), x.data_ptr(), w.data_ptr(), stats.data_ptr(), None,
                               dx_ref.data_ptr(), dw_ref.data_ptr(), db_ref.data_ptr(), scratch.data_ptr(),
                               accumulate, rows, d, stream) == 0
        ex, ew, eb = _torch_reference(rms, x, w, dy)
        # allocation-free entry point: outputs are allocated here, before the call
        dx, dw, db = torch.empty_like(x), start_w.clone(), start_b.clone()
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        assert lib.dd_norm_bwd_noalloc(rms, dy.data_ptr(), x.data_ptr(), w.data_ptr(), stats.data_ptr(),
                                       dx.data_ptr(), dw.data_ptr() if want_w else None,
                                       db.data_ptr() if want_w else None, accumulate, rows, d, stream) == 0
        torch.cuda.synchronize()
        if call > 0:        # (the very first call on a device may load the kernels' module)
            assert torch.cuda.mem_get_info()[0] == free_before, "the call changed the free device memory"
        # same arithmetic per row: dx agrees with the regular entry point to rounding
        _close(dx, dx_ref, 1e-6)
        _close(dx, ex, 1e-2)          # bf16 output against the fp32 restatement
        if want_w:
            _close(dw, dw_ref, 1e-4)  # different number of partial sums, fp32
            _close(db, db_ref, 1e-4)
            if not accumulate:
                _close(dw, ew, 5e-3)
                _close(db, eb, 5e-3)
            else:
                _close(dw - start_w, ew, 5e-3)
                _close(db - start_b, eb, 5e-3)
        else:
            assert torch.equal(dw, start_w) and torch.equal(db, start_b)


def test_norm_bwd_noalloc_refuses_bad_arguments_before_launching():
    lib = _lib()
    stream = torch.cuda.current_stream().cuda_stream
    t = torch.zeros(4 * 64 + 8, device="cuda", dtype=torch.bfloat16)
    st = torch.zeros(4, 2, device="cuda")
    ok = t.data_ptr()
    # sizes beyond the built-in scratch
    too_wide = lib.dd_norm_bwd_noalloc_max_d() + 8
    assert lib.dd_norm_bwd_noalloc(1, ok, ok, ok, st.data_ptr(), ok, None, None, 0, 4, too_wide, stream) == 1003
    assert lib.dd_norm_bwd_noalloc(1, ok, ok, ok, st.data_ptr(), ok, None, None, 0, 4, 60, stream) == 1001
    # null and misaligned pointers
    assert lib.dd_norm_bwd_noalloc(1, None, ok, ok, st.data_ptr(), ok, None, None, 0, 4, 64, stream) == 1001
    assert lib.dd_norm_bwd_noalloc(1, ok, ok, ok, None, ok, None, None, 0, 4, 64, stream) == 1001
    assert lib.dd_norm_bwd_noalloc(1, ok, ok + 2, ok, st.data_ptr(), ok, None, None, 0, 4, 64, stream) == 1002
    assert lib.dd_norm_bwd_noalloc(1, ok, ok, ok, st.data_ptr() + 4, ok, None, None, 0, 4, 64, stream) == 1002
    torch.cuda.synchronize()
