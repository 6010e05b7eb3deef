"""Llama-3-8B-shape configuration (32 layers, d=4096, 32 heads / 8 KV heads,
SwiGLU FFN 14336, RMSNorm, RoPE, vocab 128256) and scaled-down variants."""
from .decoder import Decoder, DecoderConfig, ParallelLayout  # noqa: F401


def llama3_8b(**overrides) -> DecoderConfig:
    cfg = DecoderConfig(vocab_size=128256, d_model=4096, n_layers=32, n_heads=32, n_kv_heads=8, ffn_dim=14336,
                        max_seq=4096, norm="rms", activation="swiglu", rope=True, rope_theta=500000.0, bias=False,
                        eps=1e-5)
    for k, v in overrides.items():
        setattr(cfg, k, v)
    return cfg


def llama_tiny(**overrides) -> DecoderConfig:
    """Same architecture at toy size (tests, smoke runs)."""
    cfg = DecoderConfig(vocab_size=1000, d_model=256, n_layers=2, n_heads=4, n_kv_heads=2, ffn_dim=512,
                        max_seq=256, norm="rms", activation="swiglu", rope=True, rope_theta=10000.0, bias=False)
    for k, v in overrides.items():
        setattr(cfg, k, v)
    return cfg
