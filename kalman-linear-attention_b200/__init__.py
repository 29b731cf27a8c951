"""kla-b200: a B200 (sm_100a) backend for the Kalman Linear Attention scan.

One hot path of the reference package ``kla`` -- ``kla_scan`` forward and
backward and the decode step ``kla_step`` -- as hand-written CUDA kernels behind
a C-ABI shared library, wrapped in the reference's backend-callable contract.

    import kla_b200                       # alias of this package
    y, y_var, state = kla_b200.kla_scan_b200(v, lambda_v, k, q, a, p)
    kla_b200.register()                   # kla_scan(..., backend="b200") from now on
"""

from .ops import KLAState, init_state, kla_scan_b200, kla_step_b200  # noqa: F401
from .register import register, unregister  # noqa: F401
from . import shard  # noqa: F401
from . import seqshard  # noqa: F401
from .seqshard import kla_scan_seq_sharded  # noqa: F401
from .rawscan import affine_scan_b200, mobius_scan_b200  # noqa: F401
from .decode import LayerDecoder, ModelDecoder  # noqa: F401
from . import layer  # noqa: F401
from .layer import fused_forward  # noqa: F401
from .hostpipe import scan_fwd_bwd_host  # noqa: F401
from ._lib import LIB_PATH, LibraryMissing, SYMBOLS  # noqa: F401
from .build import build  # noqa: F401

__version__ = "0.1.0"
