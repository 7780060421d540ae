"""mlx_turboquant_b200: TurboQuant KV-cache compression and attention over the compressed cache
as hand-written sm_100a CUDA kernels, behind the operator surface of alex-rentel/mlx-turboquant.

Public names follow the reference (mlx_turboquant/__init__.py:45-59).
"""

__version__ = "0.1.0"

from .cache import TurboQuantKVCache
from .patch import apply_turboquant, enable_turboquant
from .quantizer import QuantizedTensor, TurboQuantMSE, TurboQuantProd

__all__ = [
    "__version__",
    "apply_turboquant",
    "enable_turboquant",
    "TurboQuantKVCache",
    "TurboQuantMSE",
    "TurboQuantProd",
]
