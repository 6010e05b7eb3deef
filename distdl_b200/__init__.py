"""distdl_b200: a Blackwell-native partitioned-tensor parallelism framework.

Public surface (mirrors ``distdl``): ``backends``, ``config``, ``nn``,
``functional``, ``utilities``, ``logger``; plus ``ops`` (sm_100a kernels),
``parallel`` (symmetric memory, fused compute+collective kernels, FSDP / pipeline
engines), ``models`` and ``utils``.
"""
__version__ = "0.1.0"

from . import logger  # noqa: F401,E402
from . import utilities  # noqa: F401,E402
from . import backends  # noqa: F401,E402
from . import config  # noqa: F401,E402

config.set_backend()

from . import functional  # noqa: F401,E402
from . import nn  # noqa: F401,E402
