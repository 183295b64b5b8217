"""B200-native (sm_100a) sparse-attention hot path behind the H3-Optimizations
backend / projector / router protocols.

Public surface:

* ``B200SparseBackend`` - ``prepare`` / ``prepare_projected`` / ``execute``
* ``ChunkedSparseQKVProjector`` - chunked native-carrier QKV provider
* ``SparseTileRouter`` - block router (packed index list, delta LUT)
* ``HybridSparseConfig`` / ``resolve_video_budget`` - node density parameters
* ``ops`` - tensor-level wrappers over the C ABI (include/h3sparse.h)
* ``sharding`` - head partition across GPUs + NCCL all-gather
"""

from .config import HybridSparseConfig, resolve_video_budget  # noqa: F401
from .errors import (  # noqa: F401
    AttentionBackendUnavailable,
    FusedQKVError,
    SparseRouterError,
    SparseSageError,
)
from .runtime import RUNTIME_KEY, RuntimeSnapshot, runtime_options  # noqa: F401

_LAZY = {
    "B200SparseBackend": ("backend", "B200SparseBackend"),
    "preflight": ("backend", "preflight"),
    "SparseTileRouter": ("router", "SparseTileRouter"),
    "ChunkedSparseQKVProjector": ("projector", "ChunkedSparseQKVProjector"),
    "PreparedFusedQKV": ("carriers", "PreparedFusedQKV"),
}


def __getattr__(name):
    target = _LAZY.get(name)
    if target is None:
        raise AttributeError(name)
    import importlib

    module = importlib.import_module("." + target[0], __name__)
    return getattr(module, target[1])
