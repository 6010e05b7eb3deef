"""Model definitions for the benchmark configurations."""
from .decoder import Decoder, DecoderConfig, ParallelLayout, stage_layers  # noqa: F401
from .gpt2 import gpt2_tiny, gpt2_xl  # noqa: F401
from .llama import llama3_8b, llama_tiny  # noqa: F401
from .mixtral import mixtral_8x7b, mixtral_tiny  # noqa: F401
from .pipeline import PipelinedDecoder  # noqa: F401
