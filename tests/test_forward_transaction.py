"""The per-block attention transaction and its installation (host logic only).

Follows the reference's own tests of this layer, which drive ``make_forward``
with stand-in backends and projectors (tests/test_chunked_kitchen_qkv.py:260-294)
and ``configure_backend`` through a stand-in model patcher."""

from types import SimpleNamespace

import pytest
import torch

from h3_optimizations_b200.attention_forward import make_forward, rms_rope_split_half, to_hnd
from h3_optimizations_b200.patch import (H3AttentionPatchError, OWNER_MARKER, ORIGINAL_MARKER, configure_backend,
                                         installation_signature, key_for)


def test_forward_uses_original_when_runtime_projector_declines():
    calls = []

    class Projector:
        name = "declining_projector"

        @staticmethod
        def try_project(*_args, **_kwargs):
            return None

    class Backend:
        name = "must_not_run"

        @staticmethod
        def prepare_projected(*_args, **_kwargs):
            raise AssertionError("backend must not consume a declined projection")

    def original(x, rope_freqs=None, transformer_options=None):
        calls.append((x, rope_freqs, transformer_options))
        return "upstream"

    forward = make_forward(SimpleNamespace(heads=2, head_dim=4), 3, backend=Backend(), projector=Projector(),
                           fallback_forward=original)
    x, rope, options = object(), object(), {"marker": True}
    assert forward(x, rope, options) == "upstream"
    assert calls == [(x, rope, options)]
    assert forward._h3_optimizations_attention and forward._h3_optimizations_layer_index == 3
    assert forward._h3_optimizations_backend == "must_not_run"
    assert forward._h3_optimizations_projector == "declining_projector"


def _module(heads=2, seq=5):
    torch.manual_seed(0)
    hidden = heads * 128
    proj = torch.nn.Linear(hidden, 3 * hidden, bias=False)
    out_proj = torch.nn.Linear(hidden, hidden, bias=False)
    norm = lambda: SimpleNamespace(weight=torch.rand(128) + 0.5, eps=1e-6)
    return SimpleNamespace(heads=heads, head_dim=128, qkv_proj=proj, out_proj=out_proj, q_norm=norm(), k_norm=norm(),
                           forward=lambda *a, **k: "original")


def test_projected_and_unprojected_transactions():
    module = _module()
    seen = {}

    class Backend:
        name = "recording"

        def prepare_projected(self, projected, *, layer_index, transformer_options):
            seen["projected"] = (projected, layer_index)
            return "prepared-projected"

        def prepare(self, q, k, v, *, layer_index, transformer_options):
            seen["qkv"] = (q, k, v, layer_index)
            return "prepared"

        def execute(self, prepared):
            seen["executed"] = prepared
            return torch.ones(1, 2, 5, 128)

    class Projector:
        name = "chunked"

        def bind(self, bound):
            seen["bound"] = bound

        def project(self, module, x, rope, *, layer_index, transformer_options):
            return "carriers"

    x = torch.randn(5, 256)
    out = make_forward(module, 7, backend=Backend(), projector=Projector())(x)
    assert seen["bound"] is module and seen["projected"] == ("carriers", 7) and seen["executed"] == "prepared-projected"
    assert torch.equal(out, module.out_proj(torch.ones(5, 256)))

    out = make_forward(module, 2, backend=Backend())(x, None, {})
    q, k, v, layer = seen["qkv"]
    assert layer == 2 and all(tuple(t.shape) == (1, 2, 5, 128) and t.stride(-1) == 1 for t in (q, k, v))
    assert seen["executed"] == "prepared" and tuple(out.shape) == (5, 256)

    class Rank3(Backend):
        def execute(self, prepared):
            return torch.ones(2, 5, 128)

    with pytest.raises(RuntimeError, match="rank-3 output; expected HND rank 4"):
        make_forward(module, 0, backend=Rank3())(x)

    class Direct(Backend):
        def execute_projected(self, module, prepared):
            return torch.zeros(5, 256)

    assert torch.equal(make_forward(module, 0, backend=Direct(), projector=Projector())(x), torch.zeros(5, 256))
    with pytest.raises(ValueError, match="backend is required"):
        make_forward(module, 0)


def test_rms_rope_split_half_against_a_plain_restatement():
    torch.manual_seed(1)
    seq, heads = 6, 3
    x = torch.randn(seq, heads, 128).to(torch.bfloat16)
    weight = torch.rand(128) + 0.5
    angles = torch.arange(seq * 48, dtype=torch.float32).reshape(seq, 48) / 8192.0
    c, s = torch.cos(angles), torch.sin(angles)
    rope = torch.stack((c, -s, s, c), dim=-1).reshape(1, seq, 1, 48, 2, 2).to(torch.bfloat16)
    got = rms_rope_split_half(x, weight, rope, 1e-6).float()
    ref = torch.empty(seq, heads, 128)
    for t in range(seq):
        for h in range(heads):
            row = x[t, h].float()
            row = (row * torch.rsqrt((row * row).sum() / 128 + 1e-6) * weight).to(torch.bfloat16).float()
            out = row.clone()
            for d in range(48):
                f = rope[0, t, 0, d].float()
                out[d] = f[0, 0] * row[d] + f[0, 1] * row[d + 48]
                out[d + 48] = f[1, 0] * row[d] + f[1, 1] * row[d + 48]
            ref[t, h] = out.to(torch.bfloat16).float()
    assert torch.equal(got, ref)
    plain = rms_rope_split_half(x, weight, None, 1e-6)
    assert torch.equal(plain[..., 96:], got.to(torch.bfloat16)[..., 96:])  # channels 96.. are only normalised
    q, k, v = to_hnd(x, x, x)
    assert tuple(q.shape) == (1, heads, seq, 128) and q.stride(-1) == 1


class _Patcher:
    def __init__(self, blocks):
        self.model = SimpleNamespace(diffusion_model=SimpleNamespace(blocks=blocks))
        self.object_patches = {}
        self.model_options = {}

    def add_object_patch(self, key, value):
        self.object_patches[key] = value


def test_configure_backend_installs_reconciles_and_refuses_conflicts():
    blocks = [SimpleNamespace(attn=_module()) for _ in range(3)]
    patcher = _Patcher(blocks)
    backend = SimpleNamespace(name="b200", installation_signature=("b200", 1))
    assert configure_backend(patcher, backend) == (backend, 3)
    forwards = [patcher.object_patches[key_for(i)] for i in range(3)]
    assert all(getattr(f, OWNER_MARKER) for f in forwards)
    assert getattr(forwards[1], ORIGINAL_MARKER)() == "original"
    assert patcher.model_options["transformer_options"]["h3_optimizations_attention_backend"] == "b200"
    assert configure_backend(patcher, backend) == (backend, 0)  # same signature: nothing to do
    other = SimpleNamespace(name="b200", installation_signature=("b200", 2))
    assert configure_backend(patcher, other, projector_fallback_to_original=True) == (other, 3)
    assert getattr(patcher.object_patches[key_for(0)], ORIGINAL_MARKER)() == "original"  # original survives a replace

    foreign = _Patcher([SimpleNamespace(attn=_module())])
    foreign.object_patches[key_for(0)] = lambda *a, **k: None
    with pytest.raises(H3AttentionPatchError, match="another patch already owns"):
        configure_backend(foreign, backend)
    with pytest.raises(H3AttentionPatchError, match="missing out_proj"):
        broken = _module()
        del broken.out_proj
        configure_backend(_Patcher([SimpleNamespace(attn=broken)]), backend)
    with pytest.raises(H3AttentionPatchError, match="no main blocks"):
        configure_backend(_Patcher([]), backend)
    with pytest.raises(TypeError):
        configure_backend(patcher, None)
    assert installation_signature(None) is None
    assert installation_signature(SimpleNamespace(name="x"))[2] == "x"
