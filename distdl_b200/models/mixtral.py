"""Mixtral-8x7B-shape configuration (32 layers, d=4096, 32 heads / 8 KV heads,
8 experts with SwiGLU FFN 14336, top-2 softmax router, RMSNorm, vocab 32000)."""
from .decoder import Decoder, DecoderConfig, ParallelLayout  # noqa: F401


def mixtral_8x7b(**overrides) -> DecoderConfig:
    cfg = DecoderConfig(vocab_size=32000, d_model=4096, n_layers=32, n_heads=32, n_kv_heads=8, ffn_dim=14336,
                        max_seq=4096, norm="rms", activation="swiglu", rope=True, rope_theta=1000000.0, bias=False,
                        eps=1e-5, n_experts=8, top_k=2)
    for k, v in overrides.items():
        setattr(cfg, k, v)
    return cfg


def mixtral_tiny(**overrides) -> DecoderConfig:
    cfg = DecoderConfig(vocab_size=1000, d_model=256, n_layers=2, n_heads=4, n_kv_heads=2, ffn_dim=512, max_seq=256,
                        norm="rms", activation="swiglu", rope=True, rope_theta=10000.0, bias=False, n_experts=4,
                        top_k=2)
    for k, v in overrides.items():
        setattr(cfg, k, v)
    return cfg
