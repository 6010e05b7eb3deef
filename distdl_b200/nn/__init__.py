"""Distributed layers (``src/distdl/nn/__init__.py`` in the reference)."""
from .all_gather import AllGather  # noqa: F401
from .all_sum_reduce import AllSumReduce  # noqa: F401
from .broadcast import Broadcast  # noqa: F401
from .halo_exchange import HaloExchange  # noqa: F401
from .module import Module, reset_setup  # noqa: F401
from .reduce_scatter import ReduceScatter  # noqa: F401
from .repartition import Repartition  # noqa: F401
from .sum_reduce import SumReduce  # noqa: F401
from .transpose import DistributedTranspose  # noqa: F401
from . import init  # noqa: F401,E402
from .embedding import DistributedEmbedding  # noqa: F401,E402
from .embedding_zero import DistributedEmbeddingZero  # noqa: F401,E402
from .layernorm import DistributedLayerNorm  # noqa: F401,E402
from .layernorm_zero import DistributedLayerNormZero  # noqa: F401,E402
from .linear import DistributedLinear  # noqa: F401,E402
from .linear_ag import DistributedLinearAllGather  # noqa: F401,E402
from .linear_ag_zero import DistributedLinearAllGatherZero  # noqa: F401,E402
from .linear_rs import DistributedLinearReduceScatter  # noqa: F401,E402
from .linear_rs_zero import DistributedLinearReduceScatterZero  # noqa: F401,E402
from .rmsnorm_zero import DistributedRMSNormZero  # noqa: F401,E402
from . import loss  # noqa: F401,E402
from .batchnorm import DistributedBatchNorm  # noqa: F401,E402
from .conv_feature import (DistributedFeatureConv1d, DistributedFeatureConv2d, DistributedFeatureConv3d,  # noqa: F401,E402
                           DistributedFeatureConvTranspose1d, DistributedFeatureConvTranspose2d,
                           DistributedFeatureConvTranspose3d)
from .loss import (DistributedBCELoss, DistributedBCEWithLogitsLoss, DistributedKLDivLoss,  # noqa: F401,E402
                   DistributedL1Loss, DistributedMSELoss, DistributedPoissonNLLLoss)
from .pooling import (DistributedAvgPool1d, DistributedAvgPool2d, DistributedAvgPool3d,  # noqa: F401,E402
                      DistributedMaxPool1d, DistributedMaxPool2d, DistributedMaxPool3d)
from .linear_ag_expert import DistributedExpertAllGather  # noqa: F401,E402
from .linear_rs_expert import DistributedExpertReduceScatter  # noqa: F401,E402
from .conv import DistributedConv1d, DistributedConv2d, DistributedConv3d  # noqa: F401,E402
from .conv_channel import DistributedChannelConv1d, DistributedChannelConv2d, DistributedChannelConv3d  # noqa: F401,E402
from .conv_general import DistributedGeneralConv1d, DistributedGeneralConv2d, DistributedGeneralConv3d  # noqa: F401,E402
from .conv_channel_ag import (DistributedChannelAllGatherConv1d, DistributedChannelAllGatherConv2d,  # noqa: F401,E402
                              DistributedChannelAllGatherConv3d, DistributedChannelAllGatherConvTranspose1d,
                              DistributedChannelAllGatherConvTranspose2d, DistributedChannelAllGatherConvTranspose3d)
from .conv_channel_rs import (DistributedChannelReduceScatterConv1d, DistributedChannelReduceScatterConv2d,  # noqa: F401,E402
                              DistributedChannelReduceScatterConv3d, DistributedChannelReduceScatterConvTranspose1d,
                              DistributedChannelReduceScatterConvTranspose2d,
                              DistributedChannelReduceScatterConvTranspose3d)
from . import mixins  # noqa: F401,E402
from .interpolate import Interpolate  # noqa: F401,E402
from .upsampling import DistributedUpsample  # noqa: F401,E402

__all__ = [
    "AllGather", "AllSumReduce", "Broadcast", "DistributedBatchNorm", "DistributedConv1d", "DistributedConv2d",
    "DistributedConv3d", "DistributedChannelConv1d", "DistributedChannelConv2d", "DistributedChannelConv3d",
    "DistributedFeatureConv1d", "DistributedFeatureConv2d", "DistributedFeatureConv3d",
    "DistributedFeatureConvTranspose1d", "DistributedFeatureConvTranspose2d", "DistributedFeatureConvTranspose3d",
    "DistributedChannelReduceScatterConv1d", "DistributedChannelReduceScatterConv2d",
    "DistributedChannelReduceScatterConv3d", "DistributedChannelReduceScatterConvTranspose1d",
    "DistributedChannelReduceScatterConvTranspose2d", "DistributedChannelReduceScatterConvTranspose3d",
    "DistributedChannelAllGatherConv1d", "DistributedChannelAllGatherConv2d", "DistributedChannelAllGatherConv3d",
    "DistributedChannelAllGatherConvTranspose1d", "DistributedChannelAllGatherConvTranspose2d",
    "DistributedChannelAllGatherConvTranspose3d", "DistributedGeneralConv1d", "DistributedGeneralConv2d",
    "DistributedGeneralConv3d", "HaloExchange", "DistributedEmbeddingZero", "DistributedEmbedding",
    "DistributedLayerNormZero", "DistributedLayerNorm", "DistributedRMSNormZero", "DistributedLinear",
    "DistributedLinearAllGather", "DistributedLinearAllGatherZero", "DistributedLinearReduceScatter",
    "DistributedLinearReduceScatterZero", "DistributedExpertAllGather", "DistributedExpertReduceScatter",
    "DistributedL1Loss", "DistributedMSELoss", "DistributedPoissonNLLLoss", "DistributedBCELoss",
    "DistributedBCEWithLogitsLoss", "DistributedKLDivLoss", "Module", "DistributedAvgPool1d", "DistributedAvgPool2d",
    "DistributedAvgPool3d", "DistributedMaxPool1d", "DistributedMaxPool2d", "DistributedMaxPool3d", "Repartition",
    "ReduceScatter", "SumReduce", "DistributedTranspose", "Interpolate", "DistributedUpsample", "loss",
]

# beyond the reference's 64 names: attention over a sequence-split tensor (kept out of
# ``__all__`` so that the list above stays the reference's)
from .attention import DistributedSelfAttention  # noqa: E402,F401
from .ring_attention import DistributedRingAttention  # noqa: E402,F401
from .window_attention import DistributedSlidingWindowAttention  # noqa: E402,F401
