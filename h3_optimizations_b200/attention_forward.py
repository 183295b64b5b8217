"""The attention-module transaction that calls the hot path.

Mirror of the reference's ``make_forward`` (attention_forward.py:131-246): one
closure per DiT block that replaces ``block.attn.forward``.  With a projector
installed the activations go ``projector.project -> backend.prepare_projected
-> backend.execute[_projected] -> out_proj`` and never exist as floating-point
Q/K/V; without one (or when the projector declines and no fallback was given)
the module's own ``qkv_proj`` runs, Q and K get the RMS norm and the split-half
rotation, and the HND views go through ``backend.prepare`` / ``execute``.

The module must expose ``qkv_proj, q_norm, k_norm, out_proj, heads, head_dim``
(patch.py:13-20).  Control flow, argument names, the markers left on the
closure and the error texts follow the reference; the reference's dense
``attention=`` arm and its ``AttentionBackendUnavailable`` fallback to a dense
kernel do not exist here (this package has exactly one backend and no dense
path), so ``backend`` is required.
"""

from __future__ import annotations

import torch

ROPE_DIM = 96  # 48 frequency pairs: channels [0,48) rotate against [48,96), [96,128) pass through


def rms_rope_split_half(values, norm_weight, rope_freqs, epsilon):
    """RMS norm over the 128 channels of every (token, head) followed by the
    split-half rotation, with the roundings of the reference's fused epilogue
    (fused_qkv.py:230-289): the input is taken as already rounded to bf16, the
    normalised value is rounded to bf16, the rotated value is rounded to bf16.

    ``values``: ``(S, H, 128)``; ``rope_freqs``: ``(1, S, 1, 48, 2, 2)`` or
    ``None``.  Returns ``(S, H, 128)`` in the input dtype.  Runs wherever the
    tensors live; it is module glue for the unprojected entry, the projected
    entry applies the same arithmetic inside the GEMM epilogue."""
    x = values.float()
    inverse_rms = torch.rsqrt((x * x).sum(dim=-1, keepdim=True) / x.shape[-1] + float(epsilon))
    x = (x * inverse_rms * norm_weight.float()).to(torch.bfloat16).float()
    if rope_freqs is not None:
        pairs = rope_freqs.shape[-3]
        f = rope_freqs.reshape(rope_freqs.shape[1], 1, pairs, 2, 2).float()
        first, second = x[..., :pairs], x[..., pairs : 2 * pairs]
        rotated_first = f[..., 0, 0] * first + f[..., 0, 1] * second
        rotated_second = f[..., 1, 0] * first + f[..., 1, 1] * second
        x = torch.cat([rotated_first, rotated_second, x[..., 2 * pairs :]], dim=-1).to(torch.bfloat16).float()
    return x.to(values.dtype)


def finish_qkv_projection(module, projected, rope_freqs):
    """Split ``(S, 3*H*128)`` into per-head Q, K, V ``(S, H, 128)`` and apply
    the Q/K norm (+ rotation) - attention_forward.py:10-48."""
    seq = projected.shape[0]
    inner = module.heads * module.head_dim
    q, k, v = projected.split(inner, dim=-1)
    shape = (seq, module.heads, module.head_dim)
    q = rms_rope_split_half(q.reshape(shape), module.q_norm.weight.to(projected.device), rope_freqs, module.q_norm.eps)
    k = rms_rope_split_half(k.reshape(shape), module.k_norm.weight.to(projected.device), rope_freqs, module.k_norm.eps)
    return q, k, v.reshape(shape)


def project_qkv(module, x, rope_freqs):
    return finish_qkv_projection(module, module.qkv_proj(x), rope_freqs)


def to_hnd(q, k, v):
    """``(S, H, 128)`` -> HND ``(1, H, S, 128)`` strided views (attention_forward.py:55-60)."""
    return (q.transpose(0, 1).unsqueeze(0), k.transpose(0, 1).unsqueeze(0), v.transpose(0, 1).unsqueeze(0))


def _backend_name(backend):
    return getattr(backend, "name", type(backend).__name__)


def _project_or_none(projector, module, x, rope_freqs, *, layer_index, transformer_options):
    callback = getattr(projector, "try_project", None)
    if callback is None:
        callback = projector.project
    return callback(module, x, rope_freqs, layer_index=layer_index, transformer_options=transformer_options)


def _hnd_to_rows(out_hnd, module, backend):
    if out_hnd.ndim != 4:
        raise RuntimeError("%s returned rank-%d output; expected HND rank 4" % (_backend_name(backend), out_hnd.ndim))
    out = out_hnd.transpose(1, 2).reshape(out_hnd.shape[0], out_hnd.shape[2], module.heads * module.head_dim)
    return module.out_proj(out.squeeze(0))


def _finish_projected(module, backend, prepared):
    execute_projected = getattr(backend, "execute_projected", None)
    if execute_projected is not None:
        direct = execute_projected(module, prepared)
        if direct is not None:
            if direct.ndim != 2:
                raise RuntimeError("%s returned rank-%d direct projected output; expected rank 2"
                                   % (_backend_name(backend), direct.ndim))
            return direct
    return _hnd_to_rows(backend.execute(prepared), module, backend)


def make_forward(module, layer_index, backend=None, projector=None, fallback_forward=None):
    """Build the replacement for ``module.forward`` of DiT block ``layer_index``."""
    if backend is None:
        raise ValueError("a backend is required: this package has no dense attention arm")
    bind_projector = getattr(projector, "bind", None)
    if bind_projector is not None:
        bind_projector(module)

    def forward(x, rope_freqs=None, transformer_options=None):
        transformer_options = transformer_options if transformer_options is not None else {}
        if projector is not None:
            projected = _project_or_none(projector, module, x, rope_freqs, layer_index=layer_index,
                                         transformer_options=transformer_options)
            if projected is not None:
                prepared = backend.prepare_projected(projected, layer_index=layer_index,
                                                     transformer_options=transformer_options)
                del projected
                try:
                    return _finish_projected(module, backend, prepared)
                finally:
                    del prepared
            if fallback_forward is not None:
                return fallback_forward(x, rope_freqs=rope_freqs, transformer_options=transformer_options)

        q, k, v = to_hnd(*project_qkv(module, x, rope_freqs))
        prepared = backend.prepare(q, k, v, layer_index=layer_index, transformer_options=transformer_options)
        del q, k, v
        try:
            out_hnd = backend.execute(prepared)
        finally:
            del prepared
        return _hnd_to_rows(out_hnd, module, backend)

    forward._h3_optimizations_attention = True
    forward._h3_optimizations_layer_index = int(layer_index)
    forward._h3_optimizations_backend = getattr(backend, "name", None)
    forward._h3_optimizations_projector = getattr(projector, "name", None)
    return forward
