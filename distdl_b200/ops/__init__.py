"""Hand-written sm_100a operators (and their CPU stand-ins for plumbing tests)."""
from .attention import attention, attention_backward, attention_forward, attention_packed  # noqa: F401
from .activation import gelu, rope_, rope_table, swiglu  # noqa: F401
from .embedding import embedding  # noqa: F401
from .gemm import gemm, linear, matmul  # noqa: F401
from .loss import cross_entropy_  # noqa: F401
from .norm import add_layer_norm, add_rms_norm, layer_norm, rms_norm  # noqa: F401
from .optim import adamw_step_, sumsq_  # noqa: F401
