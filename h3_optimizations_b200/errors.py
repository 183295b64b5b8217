"""Typed errors of the sparse path (reference: attention/sparse/router.py:14,
sparse_sage.py:12, fused_qkv.py:26, attention/__init__.py:6)."""


class SparseRouterError(RuntimeError):
    """Invalid layout, budget or summaries handed to the tile router."""


class SparseSageError(RuntimeError):
    """Carrier / backend contract violation or kernel failure."""


class FusedQKVError(RuntimeError):
    """Chunked QKV projection contract violation."""


class AttentionBackendUnavailable(RuntimeError):
    """Raised at install time only; the one error that may trigger a dense fallback."""
