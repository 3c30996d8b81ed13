"""Bavutar's configuration reader and what the model asks of the cache manager (no GPU)."""
import copy

import pytest
import torch

import sparseengine_b200.models  # noqa: F401
from sparseengine_b200.config.registry import load_model_spec
from sparseengine_b200.engine.model import Model

CFG = {
    "architecture": "Bavutar", "vocab": 100, "width": 64, "postln_alpha": 1.5, "embedding": {"scale": 4.0},
    "logit_softcap": 20.0, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 32, "scale": 0.3,
                                        "q_temp": {"coef": 0.25, "every": 32}}, "mlp": {"kind": "dense", "ff": 128}},
        {"type": "mamba2", "mixer": {"heads": 4, "vdim": 8, "state": 16, "groups": 2, "conv": 3, "norm_groups": 2}, "mlp": None},
        {"type": "channel_delta", "mixer": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 16, "conv": 4, "rank": 5},
         "mlp": {"kind": "dense", "ff": 96}},
        {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 32, "kv_from": 0}, "mlp": None},
    ],
}


def test_the_configuration_becomes_parts_with_its_own_constants():
    typed, spec = load_model_spec(copy.deepcopy(CFG))
    assert spec.architecture == "Bavutar" and spec.residual_stream == "float32"
    assert spec.embed_scale == 4.0 and spec.logit_softcap == 20.0 and spec.vocab_size == 100
    a, s, d, b = (ls.mixer for ls in spec.layers)
    assert (a.kind, a.prep, a.v_head_dim, a.scale, a.q_temperature, a.own_kv) == ("attention", "general", 32, 0.3, (0.25, 32), True)
    assert (s.kind, s.state_size, s.groups, s.conv_taps, s.norm_groups) == ("mamba2", 16, 2, 3, 2)
    assert (d.kind, d.decay_rank, d.gate_rank, d.conv_taps) == ("channel_delta", 5, 5, 4)
    assert not b.own_kv and b.q_temperature is None and b.scale == 16 ** -0.5
    assert [ls.feed_forward is None for ls in spec.layers] == [False, True, False, True]
    assert all(ls.arrangement == "post_norm" and ls.residual_scale == 1.5 for ls in spec.layers)
    assert spec.layers[0].mixer_norm.kind == "layer_norm" and spec.layers[0].mixer_norm.eps == 1e-5
    assert [(e.cache, e.write_cache) for e in spec.order] == [(None, True), (None, True), (None, True), (0, False)]


def test_cache_needs_and_parameters():
    _, spec = load_model_spec(copy.deepcopy(CFG))
    m = Model(spec, torch.bfloat16)
    (req, layers), = m.layout.groups
    assert (req.num_kv_heads, req.head_dim, req.value_dim, layers) == (2, 16, 32, 1)
    assert m.layout.entries[3].cache_layer == m.layout.entries[0].cache_layer and not m.layout.entries[3].write
    ssm_state, delta_state = m.layout.states
    assert ssm_state.shape == (4 * 8 * 16 + 2 * (32 + 2 * 2 * 16),) and ssm_state.dtype == torch.float32
    assert delta_state.shape == (4 * 16 * 8 + 3 * (2 * 16 + 64),)
    names = {s.name for p in m.params() for s in p.sources}
    assert {"embed", "head", "final.norm", "final.norm.b", "l0.mix.q.norm", "l0.mix.k.norm", "l1.mix.conv.b", "l2.mix.a2",
            "l2.mix.v.conv", "l3.mix.q", "l0.norm2.b"} <= names
    assert not {"l3.mix.k", "l3.mix.v", "l3.mix.k.norm", "l1.norm2", "l3.norm2"} & names
    shapes = {p.qualified: tuple(p.spec.shape) for p in m.params()}
    assert shapes["layers.0.mixer.qkv"] == (4 * 16 + 2 * 16 + 2 * 32, 64) and shapes["layers.3.mixer.qkv"] == (64, 64)
    assert shapes["layers.0.mixer.o"] == (64, 4 * 32)
    assert shapes["layers.2.mixer.in_proj"] == (2 * 16 + 64 + 4 + 5 + 5, 64)


@pytest.mark.parametrize("change, text", [
    (lambda c: c["layers"][3]["mixer"].update(kv_from=1), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=3), "kv_from"),
    (lambda c: c["layers"][1].update(type="lstm"), "unknown mixer type"),
    (lambda c: c["layers"][2]["mixer"].pop("rank"), "ranks"),
    (lambda c: c["layers"][1]["mixer"].pop("state"), "missing mixer keys"),
    (lambda c: c["layers"][0].update(mlp={"kind": "moe", "ff": 8}), "feed-forward"),
    (lambda c: c.pop("vocab"), "vocab"),
])
def test_configurations_that_are_refused(change, text):
    c = copy.deepcopy(CFG)
    change(c)
    with pytest.raises(ValueError, match=text):
        load_model_spec(c)


def test_sizes_the_kernels_do_not_take_are_refused_when_the_part_is_built():
    c = copy.deepcopy(CFG)
    c["layers"][1]["mixer"]["state"] = 1024
    _, spec = load_model_spec(c)
    with pytest.raises(ValueError, match="state_size"):
        Model(spec, torch.float32)
    c = copy.deepcopy(CFG)
    c["layers"][1]["mixer"]["groups"] = 3
    _, spec = load_model_spec(c)
    with pytest.raises(ValueError, match="multiple of groups"):
        Model(spec, torch.float32)
