"""tcgen05 GEMM against a plain fp32 PyTorch reference of the same product."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, b):
    return a.float() @ b.float().transpose(-1, -2)


def _check(out, ref, tol=2e-2):
    err = (out.float() - ref).abs().max().item()
    scale = ref.abs().max().item() + 1e-6
    assert err / scale < tol, f"max err {err} vs scale {scale}"


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (200, 600, 1600), (4096, 3072, 4096),
                                   (77, 88, 96), (1024, 1024, 8), (130, 264, 72)])
@pytest.mark.parametrize("a_mn,b_mn", [(0, 0), (0, 1), (1, 0), (1, 1)])
def test_gemm_layouts(M, N, K, a_mn, b_mn):
    from distdl_b200 import _native
    from distdl_b200.ops import gemm
    torch.manual_seed(0)
    dev = "cuda"
    # leading dimensions must be multiples of 8 elements: pad the storage
    def make(rows, cols, mn):
        if mn:
            ld = (rows + 7) // 8 * 8
            st = torch.randn(cols, ld, device=dev, dtype=torch.bfloat16)
            return st[:, :rows].t()
        ld = (cols + 7) // 8 * 8
        st = torch.randn(rows, ld, device=dev, dtype=torch.bfloat16)
        return st[:, :cols]
    a = make(M, K, a_mn)
    b = make(N, K, b_mn)
    out = gemm(a, b)
    torch.cuda.synchronize()
    assert _native.read_status()[0] == 0
    _check(out, _ref(a, b))


def test_gemm_bias_accumulate_fp32():
    from distdl_b200.ops import gemm
    torch.manual_seed(1)
    M, N, K = 512, 768, 320
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    bias = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    out = gemm(a, b, bias=bias)
    _check(out, _ref(a, b) + bias.float())
    acc = torch.randn(M, N, device="cuda", dtype=torch.float32)
    ref = acc.clone() + _ref(a, b)
    gemm(a, b, out=acc, accumulate=True)
    _check(acc, ref, tol=1e-3)
    accb = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    refb = accb.float() + _ref(a, b)
    gemm(a, b, out=accb, accumulate=True)
    _check(accb, refb)


def test_gemm_batched():
    from distdl_b200.ops import gemm
    torch.manual_seed(2)
    B, M, N, K = 5, 256, 384, 128
    a = torch.randn(B, M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(B, N, K, device="cuda", dtype=torch.bfloat16)
    out = gemm(a, b)
    _check(out, _ref(a, b))
    bt = torch.randn(B, K, N, device="cuda", dtype=torch.bfloat16)
    out = gemm(a, bt.transpose(1, 2))
    _check(out, a.float() @ bt.float())


def test_linear_autograd_matches_torch():
    from distdl_b200.ops import linear
    torch.manual_seed(3)
    x = torch.randn(4, 96, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(512, 256, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_()
    b = torch.randn(512, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = linear(x, w, b)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr = x.detach().float().requires_grad_()
    wr = w.detach().float().requires_grad_()
    br = b.detach().float().requires_grad_()
    yr = torch.nn.functional.linear(xr, wr, br)
    yr.backward(dy.float())
    _check(y, yr)
    _check(x.grad, xr.grad)
    _check(w.grad, wr.grad)
    _check(b.grad, br.grad)


@pytest.mark.parametrize("M,N,K", [(256, 512, 4096), (384, 256, 8192), (1024, 768, 1600), (512, 512, 14336)])
def test_gemm_error_bound_scales_with_the_contraction_length(M, N, K):
    """Element-wise bounds that a lost k-block cannot hide behind.  With fp32 output the only error is
    the accumulation's: a few fp32 roundings of sums of size sqrt(K), orders of magnitude below the
    sqrt(64) / sqrt(K) share of one 64-deep k-block.  With bf16 output every element is within one
    bf16 rounding of the exact value (plus the same accumulation term)."""
    from distdl_b200.ops import gemm
    torch.manual_seed(K)
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    ref = a.double() @ b.double().t()
    acc_term = 1e-4 * (K ** 0.5)                  # generous for fp32 accumulation in any order; one lost k-block is ~ 8
    out32 = gemm(a, b, out_dtype=torch.float32)
    err = (out32.double() - ref).abs().max().item()
    assert err < acc_term, (err, acc_term)
    out16 = gemm(a, b)
    bound = ref.abs() * 2.0 ** -8 + acc_term
    assert bool(((out16.double() - ref).abs() <= bound).all()), ((out16.double() - ref).abs() - bound).max().item()
    # the gradient layouts (dy @ w and dy^T @ x) under the same bound
    wg = gemm(a.t().contiguous().t(), b, out_dtype=torch.float32)          # A as a transposed (MN-major) view
    assert (wg.double() - ref).abs().max().item() < acc_term
    at = torch.randn(K, M, device="cuda", dtype=torch.bfloat16)      # MN-major operands, as in a weight gradient
    bt = torch.randn(K, N, device="cuda", dtype=torch.bfloat16)
    reft = at.double().t() @ bt.double()
    outt = gemm(at.t(), bt.t(), out_dtype=torch.float32)
    assert (outt.double() - reft).abs().max().item() < acc_term
