"""Flash attention kernels against fp32 PyTorch scaled-dot-product attention."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(q, k, v, batch, seq, causal):
    from distdl_b200.ops.attention import _reference
    return _reference(q.float(), k.float(), v.float(), batch, seq, causal, 1.0 / math.sqrt(q.shape[-1]))


@pytest.mark.parametrize("batch,seq,Hq,Hkv,D,causal", [
    (1, 128, 1, 1, 128, True), (2, 256, 4, 2, 128, True), (1, 512, 8, 2, 128, False), (2, 384, 5, 5, 64, True),
    (1, 1024, 4, 1, 128, True), (2, 512, 6, 3, 64, True), (1, 256, 2, 2, 64, False)])
def test_attention_forward(batch, seq, Hq, Hkv, D, causal):
    from distdl_b200 import _native
    from distdl_b200.ops import attention_forward
    torch.manual_seed(0)
    T = batch * seq
    qkv = torch.randn(T, Hq + 2 * Hkv, D, device="cuda", dtype=torch.bfloat16)
    q, k, v = qkv[:, :Hq], qkv[:, Hq:Hq + Hkv], qkv[:, Hq + Hkv:]
    out, lse = attention_forward(q, k, v, batch, seq, causal)
    torch.cuda.synchronize()
    assert _native.read_status()[0] == 0
    ref = _ref(q, k, v, batch, seq, causal)
    err = (out.float() - ref).abs().max().item()
    assert err < 2e-2, err
    # log-sum-exp of the scaled scores
    qh = q.float().reshape(batch, seq, Hq, D).transpose(1, 2)
    kh = k.float().reshape(batch, seq, Hkv, D).transpose(1, 2).repeat_interleave(Hq // Hkv, 1)
    s = qh @ kh.transpose(-1, -2) / math.sqrt(D)
    if causal:
        s = s.masked_fill(torch.triu(torch.ones(seq, seq, device="cuda", dtype=torch.bool), 1), float("-inf"))
    assert (torch.logsumexp(s, -1) - lse).abs().max().item() < 2e-2


@pytest.mark.parametrize("batch,seq,Hq,Hkv,D,causal", [
    (1, 128, 1, 1, 128, True), (2, 256, 4, 2, 128, True), (1, 512, 4, 1, 128, False), (2, 384, 3, 3, 64, True),
    (2, 512, 4, 2, 64, True)])
def test_attention_backward(batch, seq, Hq, Hkv, D, causal):
    from distdl_b200 import _native
    from distdl_b200.ops import attention
    torch.manual_seed(1)
    T = batch * seq
    qkv = torch.randn(T, Hq + 2 * Hkv, D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    q, k, v = qkv[:, :Hq], qkv[:, Hq:Hq + Hkv], qkv[:, Hq + Hkv:]
    out = attention(q, k, v, batch, seq, causal)
    dout = torch.randn_like(out)
    out.backward(dout)
    torch.cuda.synchronize()
    assert _native.read_status()[0] == 0
    ref_in = qkv.detach().float().requires_grad_()
    qr, kr, vr = ref_in[:, :Hq], ref_in[:, Hq:Hq + Hkv], ref_in[:, Hq + Hkv:]
    ref = _ref(qr, kr, vr, batch, seq, causal)
    ref.backward(dout.float())
    for name, sl in (("dq", slice(0, Hq)), ("dk", slice(Hq, Hq + Hkv)), ("dv", slice(Hq + Hkv, None))):
        g, gr = qkv.grad[:, sl].float(), ref_in.grad[:, sl]
        err = (g - gr).abs().max().item()
        scale = gr.abs().max().item()
        assert err / scale < 3e-2, f"{name}: err {err} scale {scale}"
