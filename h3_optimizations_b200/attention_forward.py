"""The attention-module transaction that calls the hot path.

Takes the place of the reference's ``make_forward`` (attention_forward.py:131-246):
one replacement for ``block.attn.forward`` per DiT block.  The contract kept is
the call signature ``forward(x, rope_freqs=None, transformer_options=None)``,
the backend / projector protocols it drives, the marker attributes left on the
returned function and the error texts.  The transaction itself is an object
(``AttentionTransaction``) with one method per route through the block:

* ``projected``: ``projector.[try_]project -> backend.prepare_projected ->
  backend.execute_projected | execute -> out_proj``; the activations never
  exist as floating-point Q/K/V;
* ``unprojected``: the module's own ``qkv_proj``, RMS norm and split-half
  rotation of Q and K, HND views through ``backend.prepare`` / ``execute``.

A projector that declines (``try_project`` returns ``None``) hands the call to
the fallback forward when one was given, else to the unprojected route.  The
reference's dense ``attention=`` arm and its fallback to a dense kernel do not
exist here (this package has exactly one backend), so ``backend`` is required.
The module must expose ``qkv_proj, q_norm, k_norm, out_proj, heads, head_dim``
(patch.py:13-20).
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
    return tuple(t.transpose(0, 1).unsqueeze(0) for t in (q, k, v))


class AttentionTransaction:
    """One block's attention call.  Holds the module, its layer index, the
    backend and the optional projector / fallback forward."""

    def __init__(self, module, layer_index, backend, projector=None, fallback_forward=None):
        self.module = module
        self.layer_index = int(layer_index)
        self.backend = backend
        self.projector = projector
        self.fallback_forward = fallback_forward
        bind = getattr(projector, "bind", None)
        if bind is not None:
            bind(module)

    @property
    def backend_name(self):
        return getattr(self.backend, "name", type(self.backend).__name__)

    # -- the two routes ---------------------------------------------------------

    def __call__(self, x, rope_freqs=None, transformer_options=None):
        options = {} if transformer_options is None else transformer_options
        if self.projector is not None:
            carriers = self._ask_projector(x, rope_freqs, options)
            if carriers is not None:
                return self.projected(carriers, options)
            if self.fallback_forward is not None:
                return self.fallback_forward(x, rope_freqs=rope_freqs, transformer_options=options)
        return self.unprojected(x, rope_freqs, options)

    def _ask_projector(self, x, rope_freqs, options):
        ask = getattr(self.projector, "try_project", None) or self.projector.project
        return ask(self.module, x, rope_freqs, layer_index=self.layer_index, transformer_options=options)

    def projected(self, carriers, options):
        prepared = self.backend.prepare_projected(carriers, layer_index=self.layer_index, transformer_options=options)
        del carriers  # the carriers now belong to `prepared`
        rows = self._rows_from_backend(prepared)
        if rows is not None:
            return rows
        return self._out_proj(self.backend.execute(prepared))

    def _rows_from_backend(self, prepared):
        """A backend may finish the block itself and return ``(S, hidden)``."""
        finish = getattr(self.backend, "execute_projected", None)
        rows = None if finish is None else finish(self.module, prepared)
        if rows is not None and rows.ndim != 2:
            raise RuntimeError("%s returned rank-%d direct projected output; expected rank 2"
                               % (self.backend_name, rows.ndim))
        return rows

    def unprojected(self, x, rope_freqs, options):
        prepared = self.backend.prepare(*to_hnd(*project_qkv(self.module, x, rope_freqs)),
                                        layer_index=self.layer_index, transformer_options=options)
        return self._out_proj(self.backend.execute(prepared))

    def _out_proj(self, out_hnd):
        if out_hnd.ndim != 4:
            raise RuntimeError("%s returned rank-%d output; expected HND rank 4" % (self.backend_name, out_hnd.ndim))
        batch, _, sequence, _ = out_hnd.shape
        rows = out_hnd.transpose(1, 2).reshape(batch, sequence, self.module.heads * self.module.head_dim)
        return self.module.out_proj(rows.squeeze(0))


def make_forward(module, layer_index, backend=None, projector=None, fallback_forward=None):
    """Build the replacement for ``module.forward`` of DiT block ``layer_index``."""
    if backend is None:
        raise ValueError("a backend is required: this package has no dense attention arm")
    transaction = AttentionTransaction(module, layer_index, backend, projector, fallback_forward)

    def forward(x, rope_freqs=None, transformer_options=None):
        return transaction(x, rope_freqs, transformer_options)

    forward._h3_optimizations_attention = True
    forward._h3_optimizations_layer_index = int(layer_index)
    forward._h3_optimizations_backend = getattr(backend, "name", None)
    forward._h3_optimizations_projector = getattr(projector, "name", None)
    return forward
