"""Attention part of :mod:`distdl_b200.utils.kernel_bench`."""

import torch


def bench_attention(rows, time_op):
    from distdl_b200.ops import attention_backward, attention_forward
    for (batch, seq, Hq, Hkv, D) in [(1, 4096, 32, 8, 128), (4, 4096, 32, 8, 128), (16, 2048, 25, 25, 64)]:
        T = batch * seq
        qkv = torch.randn(T, Hq + 2 * Hkv, D, device="cuda", dtype=torch.bfloat16)
        q, k, v = qkv[:, :Hq], qkv[:, Hq:Hq + Hkv], qkv[:, Hq + Hkv:]
        flops = 4.0 * batch * Hq * seq * seq * D / 2
        ms = time_op(lambda: attention_forward(q, k, v, batch, seq, True))
        rows.append(f"attention fwd causal b{batch} s{seq} h{Hq}/{Hkv} d{D}: {ms:.3f} ms {flops / ms / 1e9:.1f} TFLOP/s")
        try:
            qh = q.reshape(batch, seq, Hq, D).transpose(1, 2)
            kh = k.reshape(batch, seq, Hkv, D).transpose(1, 2)
            vh = v.reshape(batch, seq, Hkv, D).transpose(1, 2)
            ms = time_op(lambda: torch.nn.functional.scaled_dot_product_attention(qh, kh, vh, is_causal=True,
                                                                                  enable_gqa=True))
            rows.append(f"   torch SDPA (library) same shape: {ms:.3f} ms {flops / ms / 1e9:.1f} TFLOP/s")
        except Exception as e:  # library path unavailable for this shape
            rows.append(f"   torch SDPA unavailable: {type(e).__name__}")
        try:
            out, lse = attention_forward(q, k, v, batch, seq, True)
            dout = torch.randn_like(out)
            ms = time_op(lambda: attention_backward(dout, q, k, v, out, lse, batch, seq, True))
            rows.append(f"attention bwd same shape: {ms:.3f} ms {2.5 * flops / ms / 1e9:.1f} TFLOP/s")
        except Exception as e:
            rows.append(f"   attention bwd not run: {type(e).__name__}: {e}")
