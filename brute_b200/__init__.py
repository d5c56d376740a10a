"""brute_b200 — the ``brute.bit1`` hot path on B200 (sm_100a).

``import brute_b200 as brute`` gives the reference's namespace: everything from
``torch``, plus ``Tensor``, ``bit1``, the bit1-aware factories, the ``fast``
helpers (which override the same-named torch functions, as in the reference),
``parallel_streams``, ``cuda_graphs``; ``torch.ops.brute.*`` is registered on
import. ``nn`` and ``optim`` are ``None`` (the reference ships neither).
"""
from torch import *  # noqa: F401,F403

from . import ops as _ops_registration  # noqa: F401  (registers torch.ops.brute.*)
from .tensor import Tensor, bit1  # noqa: E402
from .functional import (  # noqa: E402
    zeros, ones, empty, full,
    tensor, as_tensor, from_numpy,
    rand, randn, randint,
    rand_like, randn_like, zeros_like, ones_like, full_like, empty_like,
    arange, linspace, eye,
)
from .fast import *  # noqa: E402,F401,F403
from . import cuda_graphs, fast, streams  # noqa: E402
from .kernels import (binary_attention, binary_linear, host_matmul, pack_sign,  # noqa: E402
                      sharded_attention, sharded_matmul)  # noqa: E402
from .serialization import load_packed, save_packed  # noqa: E402

nn = None
optim = None
parallel_streams = streams.parallel_streams

from torch import (  # noqa: E402,F401
    linalg, fft, special, autograd, cuda, backends, distributions, utils, jit, hub, profiler, ao, fx,
)
