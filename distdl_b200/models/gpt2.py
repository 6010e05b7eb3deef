"""GPT-2-XL-shape configuration (48 layers, d=1600, 25 heads, FFN 6400, vocab
50257, LayerNorm, GELU, learned positions, biases)."""
from .decoder import Decoder, DecoderConfig, ParallelLayout  # noqa: F401


def gpt2_xl(**overrides) -> DecoderConfig:
    cfg = DecoderConfig(vocab_size=50257, d_model=1600, n_layers=48, n_heads=25, n_kv_heads=25, ffn_dim=6400,
                        max_seq=2048, norm="layer", activation="gelu", rope=False, bias=True, eps=1e-5, zero=False)
    for k, v in overrides.items():
        setattr(cfg, k, v)
    return cfg


def gpt2_tiny(**overrides) -> DecoderConfig:
    cfg = DecoderConfig(vocab_size=1000, d_model=192, n_layers=2, n_heads=3, n_kv_heads=3, ffn_dim=384, max_seq=256,
                        norm="layer", activation="gelu", rope=False, bias=True, zero=False)
    for k, v in overrides.items():
        setattr(cfg, k, v)
    return cfg
