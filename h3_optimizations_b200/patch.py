"""Install the attention transaction on every DiT block of a model.

Takes the place of the reference's ``configure_backend`` (patch.py:91-185).  The
model handle is duck-typed the way ComfyUI's ``ModelPatcher`` is used there:
``object_patches`` (dict), ``add_object_patch(key, value)``, ``model_options``
(dict) and the blocks at ``model.diffusion_model.blocks``; every block's
``attn`` must expose ``qkv_proj, q_norm, k_norm, out_proj, heads, head_dim``.

What is contract and therefore identical to the reference: the object-patch key
``diffusion_model.blocks.<i>.attn.forward``, the three marker attributes left on
an installed forward, the exception type and the ``transformer_options`` entry
naming the backend.  The installation itself is organised around one question
asked of the patch table - who holds each block's key - whose answer is one of
four states handled by ``configure_backend``.
"""

from __future__ import annotations

import logging
from dataclasses import dataclass

from .attention_forward import make_forward

OWNER_MARKER = "_h3_optimizations_attention"
SIGNATURE_MARKER = "_h3_optimizations_attention_signature"
ORIGINAL_MARKER = "_h3_optimizations_attention_original"
BLOCKS_ATTR = "diffusion_model.blocks"
REQUIRED_ATTRS = ("qkv_proj", "q_norm", "k_norm", "out_proj", "heads", "head_dim")


class H3AttentionPatchError(RuntimeError):
    pass


def key_for(index):
    return "%s.%d.attn.forward" % (BLOCKS_ATTR, int(index))


def installation_signature(value):
    """Hashable identity of a backend / projector: its own
    ``installation_signature`` (attribute or method) when it has one, else what
    can be said about a bare callable or object (patch.py:31-51)."""
    if value is None:
        return None
    own = getattr(value, "installation_signature", None)
    own = own() if callable(own) else own
    if own is not None:
        return own
    if callable(value):
        target = getattr(value, "__func__", value)
        kind = type(target)
        return (getattr(target, "__module__", kind.__module__), getattr(target, "__qualname__", kind.__qualname__),
                id(target))
    return (type(value).__module__, type(value).__qualname__, getattr(value, "name", None))


def get_blocks(model_patcher):
    node = getattr(model_patcher, "model", model_patcher)
    for name in BLOCKS_ATTR.split("."):
        node = getattr(node, name, None)
        if node is None:
            return ()
    return tuple(node)


def _check_attention(index, block):
    attn = getattr(block, "attn", None)
    if attn is None:
        raise H3AttentionPatchError("H3 block %d has no attention module" % index)
    absent = [name for name in REQUIRED_ATTRS if not hasattr(attn, name)]
    if absent:
        raise H3AttentionPatchError("H3 block %d attention is missing %s" % (index, ", ".join(absent)))
    width = getattr(attn.qkv_proj, "out_features", None)
    expected = 3 * int(attn.heads) * int(attn.head_dim)
    if width is not None and int(width) != expected:
        raise H3AttentionPatchError("H3 block %d qkv_proj projects to %d, expected %d" % (index, width, expected))
    return attn


def validate(model_patcher):
    """The attention modules of all blocks, or ``H3AttentionPatchError``."""
    blocks = get_blocks(model_patcher)
    if not blocks:
        raise H3AttentionPatchError("MiniMax H3 has no main blocks")
    return tuple(_check_attention(index, block) for index, block in enumerate(blocks))


@dataclass
class _Holder:
    """Who holds one block's patch key: nobody, this package, or someone else."""

    key: str
    patch: object  # the installed callable or None

    @property
    def ours(self):
        return self.patch is not None and bool(getattr(self.patch, OWNER_MARKER, False))

    @property
    def foreign(self):
        return self.patch is not None and not self.ours

    @property
    def signature(self):
        return getattr(self.patch, SIGNATURE_MARKER, None)

    @property
    def original(self):
        return getattr(self.patch, ORIGINAL_MARKER, None)


def _originals_to_wrap(holders, modules, wanted):
    """The forwards the new closures must keep as their originals, or ``None``
    when exactly ``wanted`` is installed already."""
    mine = [holder for holder in holders if holder.ours]
    if not mine:
        taken = next((holder.key for holder in holders if holder.foreign), None)
        if taken is not None:
            raise H3AttentionPatchError("another patch already owns %s; remove one H3 attention patch" % taken)
        return [module.forward for module in modules]
    if len(mine) != len(holders):
        raise H3AttentionPatchError("only %d of %d H3 attention blocks carry this patch" % (len(mine), len(holders)))
    if all(holder.signature == wanted for holder in mine):
        return None
    originals = [holder.original for holder in mine]
    if any(original is None for original in originals):
        raise H3AttentionPatchError("installed H3 attention patch has no recoverable original")
    return originals


def configure_backend(model_patcher, backend, projector=None, *, projector_fallback_to_original=False):
    """Install this package's attention transaction on every block, replacing an
    earlier installation of its own whose backend / projector / fallback choice
    differs.  Returns ``(backend, number of forwards (re)installed)``: zero when
    the same choice is installed already.  A key held by another package is an
    error."""
    if backend is None:
        raise TypeError("backend must not be None")
    modules = validate(model_patcher)
    table = getattr(model_patcher, "object_patches", {})
    holders = [_Holder(key_for(index), table.get(key_for(index))) for index in range(len(modules))]
    wanted = (installation_signature(backend), installation_signature(projector), bool(projector_fallback_to_original))
    originals = _originals_to_wrap(holders, modules, wanted)
    if originals is None:
        return backend, 0

    for index, (module, original) in enumerate(zip(modules, originals)):
        forward = make_forward(module, index, backend=backend, projector=projector,
                               fallback_forward=original if projector_fallback_to_original else None)
        for marker, value in ((OWNER_MARKER, True), (SIGNATURE_MARKER, wanted), (ORIGINAL_MARKER, original)):
            setattr(forward, marker, value)
        model_patcher.add_object_patch(holders[index].key, forward)

    backend_name = getattr(backend, "name", type(backend).__name__)
    options = dict(model_patcher.model_options.get("transformer_options", {}))
    options["h3_optimizations_attention_backend"] = backend_name
    model_patcher.model_options["transformer_options"] = options
    logging.info("[H3 Optimizations] resolved %d attention forwards: backend=%s projector=%s", len(modules),
                 backend_name, getattr(projector, "name", "standard_qkv"))
    return backend, len(modules)
