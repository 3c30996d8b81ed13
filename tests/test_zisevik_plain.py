"""The Zisevik design without a GPU: the plain implementation's own pieces on cases worked by hand, the
premises of the GPU tests (that a window one key off, a missing sink, or a changed far token show
in the plain logits), and what the configuration reader accepts and refuses."""
import copy

import numpy as np
import pytest
import torch

import plain_zisevik as pz
import trace_util as tu
from test_zisevik_gpu import config, dense, lat, moe, ret, sharp_window_model


def test_the_plain_mechanisms_are_what_they_claim():
    """The plain implementation's own pieces on cases that can be worked by hand."""
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0, 5.0]]], dtype=torch.float64)             # one token, one head, 4 rotated dims + 1
    y = pz.rotate_half_pairs(x, torch.tensor([3]), 4, 100.0)
    a0, a1 = 3.0, 3.0 * 100.0 ** -0.5
    want = [np.cos(a0) - 3 * np.sin(a0), 2 * np.cos(a1) - 4 * np.sin(a1), 3 * np.cos(a0) + np.sin(a0),
            4 * np.cos(a1) + 2 * np.sin(a1), 5.0]
    assert np.allclose(y[0, 0].numpy(), want)
    assert np.allclose(pz.unit_rms(torch.tensor([3.0, 4.0], dtype=torch.float64), 0.0).numpy(), [3 / 12.5 ** 0.5, 4 / 12.5 ** 0.5])
    # a router with top = experts weighs all experts by the softmax of the biased logits
    cfg = config(8, 10, [ret(1, 4, 4, (0.5,), mlp=moe(3, 3, 4))])
    w = {k: v.double() for k, v in pz.random_weights(cfg, 1).items()}
    h = torch.randn(5, 8, dtype=torch.float64)
    z = torch.softmax(h @ w["l0.mlp.router"].T + w["l0.mlp.router.b"], -1)
    each = [(pz.silu(h @ w[f"l0.mlp.e{e}.gate"].T) * (h @ w[f"l0.mlp.e{e}.up"].T)) @ w[f"l0.mlp.e{e}.down"].T for e in range(3)]
    assert torch.allclose(pz.moe_ff(h, w, "l0.mlp.", cfg["layers"][0]["mlp"]), sum(z[:, e:e + 1] * each[e] for e in range(3)))


def test_the_plain_window_and_sink_matter():
    """The premise of the test above, on the plain implementation: a window one key longer or
    shorter, or no sink, moves the logits far beyond the bounds the engine is held to."""
    cfg, w = sharp_window_model(37)
    toks = tu.random_prompt(80, 150, 60)
    ref = pz.forward(cfg, w, toks)
    rms = float(ref.pow(2).mean().sqrt())
    for other in (36, 38):
        c = copy.deepcopy(cfg)
        c["layers"][0]["mixer"]["mask"]["size"] = other
        d = pz.forward(c, w, toks) - ref
        assert float(d[:36].abs().max()) < 1e-9                     # the first tokens see everything either way
        assert float(d[40:].pow(2).mean().sqrt()) / rms > 1e-2
    no_sink = dict(w)
    no_sink["l0.mix.sink"] = torch.full_like(w["l0.mix.sink"], -1e4)
    assert float((pz.forward(cfg, no_sink, toks) - ref).pow(2).mean().sqrt()) / rms > 1e-2


def test_what_a_configuration_must_have():
    import sparseengine_b200.models  # noqa: F401  (registers the architectures)
    from sparseengine_b200.config.registry import load_model_spec
    good = config(32, 40, [lat(2, 8, 8, 8, 8, 8, 5, mlp=dense(16)), ret(2, 8, 8, (0.9, 0.8))], loop=(0, 1, 2))
    _, spec = load_model_spec(good)
    assert [(e.layer, e.reinject) for e in spec.order] == [(0, True), (0, True), (1, False)]
    assert spec.layers[0].mixer.window == 5 and spec.layers[0].mixer.sink and spec.layers[1].feed_forward is None
    for breaker, word in ((lambda c: c["layers"][0].__setitem__("type", "attention"), "unknown mixer type"),
                          (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
                          (lambda c: c["layers"][1]["mixer"].__setitem__("decay", [0.9]), "one entry per head"),
                          (lambda c: c["loop"].__setitem__("stop", 3), "does not fit"),
                          (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "gated"), "'dense' or 'moe'")):
        bad = copy.deepcopy(good)
        breaker(bad)
        with pytest.raises(ValueError, match=word):
            load_model_spec(bad)


def test_sizes_the_kernels_do_not_take_are_refused_when_the_parts_are_built():
    from sparseengine_b200.config.specs import LatentAttentionSpec, RetentionSpec, RotarySpec
    from sparseengine_b200.csrc import ops
    from sparseengine_b200.parts.base import make_mixer
    rot = RotarySpec(rotary_dim=16, theta=1e4)
    ok = dict(hidden_size=64, num_heads=2, head_dim=16, rot_dim=16, v_head_dim=16, q_rank=8, scale=0.1, position=rot)
    make_mixer(LatentAttentionSpec(kv_rank=ops.LIMITS["latent_max_row"] - 16, **ok), torch.float32)
    with pytest.raises(ValueError, match=str(ops.LIMITS["latent_max_row"])):
        make_mixer(LatentAttentionSpec(kv_rank=ops.LIMITS["latent_max_row"] - 15, **ok), torch.float32)
    with pytest.raises(ValueError, match="rotates 16 dims"):
        make_mixer(LatentAttentionSpec(kv_rank=8, **dict(ok, rot_dim=8)), torch.float32)
    most = ops.LIMITS["retention_max_head_dim"]
    make_mixer(RetentionSpec(hidden_size=64, num_heads=2, head_dim=most, v_head_dim=8, decays=(0.9, 0.8), position=rot), torch.float32)
    with pytest.raises(ValueError, match=str(most)):
        make_mixer(RetentionSpec(hidden_size=64, num_heads=2, head_dim=most + 1, v_head_dim=8, decays=(0.9, 0.8)), torch.float32)
    with pytest.raises(ValueError, match="one decay per head"):
        make_mixer(RetentionSpec(hidden_size=64, num_heads=2, head_dim=8, v_head_dim=8, decays=(0.9,)), torch.float32)
