"""bittorch_b200 — B200 (sm_100a) backend of the BitTorch ternary linear layer.

Drop-in for the hot path of the reference package ``bittorch``: the same public names
(``nn.TernaryLinear``, ``nn.TernaryLinearInference``, ``quant.ternary_quantize``,
``quant.pack_ternary_transposed``, ``ops.ternary_linear_packed_forward`` ...), computed by
hand-written CUDA kernels behind a torch-free C ABI (``include/bittorch_b200.h``).
``import bittorch_b200 as bittorch`` is the intended switch.
"""

__version__ = "0.2.0"

import torch  # noqa: F401

try:
    from . import _C
    _HAS_CUDA_EXT = True
except ImportError:  # library not built: has_cuda_ext() is False and every op raises when used
    _C = None
    _HAS_CUDA_EXT = False

from . import quant  # noqa: E402
from . import ops  # noqa: E402
from . import nn  # noqa: E402
from . import utils  # noqa: E402
from . import parallel  # noqa: E402


def has_cuda_ext() -> bool:
    """True when the CUDA library is built and loadable (bittorch/__init__.py:15-24)."""
    return _HAS_CUDA_EXT
