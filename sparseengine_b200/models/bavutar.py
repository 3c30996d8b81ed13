"""Bavutar: a decoder-only hybrid whose ``config.json`` lists its layers one by one.

Every layer is post-norm over a 32-bit stream: ``x <- LN1(a x + mixer(x))`` and, where the layer
has a feed-forward, ``x <- LN2(a x + ff(x))`` with ``a = postln_alpha`` and layer norms with
weight and bias.  A layer's mixer is one of

* ``attention``: grouped-query softmax attention without rotation; RMS norm over the whole query
  and key projections; a query temperature ``1 + coef ln(floor((p + 1) / every) + 1)``; score
  scale from the configuration; value heads of their own size; ``kv_from: j`` attends over layer
  ``j``'s cache and has no key/value tensors;
* ``mamba2``: selective state space (``parts.recurrent.StateSpaceMixer``);
* ``channel_delta``: gated delta rule with per-channel decay (``parts.recurrent.GatedDeltaMixer``).

The feed-forward is ungated with a squared relu.  The embedding is scaled, the final norm is a
layer norm, the logits are capped by ``c tanh(x / c)``.  Tensor names: ``embed``, ``head``,
``final.norm[.b]``, ``l<i>.norm1[.b]``, ``l<i>.norm2[.b]``, ``l<i>.mix.*``, ``l<i>.mlp.up|down``.
Sizes that the configuration leaves out (the ranks of the low-rank decay and gate projections)
are read from the checkpoint's tensor shapes, or from the optional mixer key ``rank`` when there
is no checkpoint (random weights).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from ..config.registry import register_architecture
from ..config.specs import (AttentionSpec, GatedDeltaSpec, LayerNormSpec, LayerSpec, ModelSpec, PlainMLPSpec,
                            ScheduleEntry, Source, StateSpaceSpec)

ARCHITECTURE = "Bavutar"
MIXER_TYPES = ("attention", "mamba2", "channel_delta")
DEFAULT_MAX_POSITION = 1 << 20      # the design has no position table; the cache manager wants a bound


@dataclass(frozen=True)
class BavutarConfig:
    vocab: int
    width: int
    layers: tuple                      # of dicts {"type", "mixer", "mlp"} as in config.json (validated)
    embedding_scale: float
    postln_alpha: float
    norm_eps: float
    logit_softcap: Optional[float]
    max_position: int
    ranks: tuple                       # per layer (decay rank, gate rank) or None
    bare_second_norm: tuple = ()       # layers without feed-forward whose checkpoint still holds a second norm

    uses_checkpoint_shapes = True

    @classmethod
    def from_dict(cls, raw: dict, shapes: Optional[dict] = None) -> "BavutarConfig":
        problems = []
        for key in ("vocab", "width", "layers"):
            if raw.get(key) is None:
                problems.append(f"missing key {key!r}")
        layers = raw.get("layers") or []
        if not isinstance(layers, list) or not layers:
            problems.append("'layers' must be a non-empty list")
            layers = []
        ranks = []
        for i, layer in enumerate(layers):
            kind, m = layer.get("type"), layer.get("mixer") or {}
            if kind not in MIXER_TYPES:
                problems.append(f"layer {i}: unknown mixer type {kind!r} (known: {', '.join(MIXER_TYPES)})")
                ranks.append(None)
                continue
            need = {"attention": ("heads", "kv_heads", "dim", "vdim"),
                    "mamba2": ("heads", "vdim", "state", "groups", "conv", "norm_groups"),
                    "channel_delta": ("heads", "kv_heads", "dim", "vdim", "conv")}[kind]
            missing = [k for k in need if m.get(k) is None]
            if missing:
                problems.append(f"layer {i} ({kind}): missing mixer keys {missing}")
            if kind == "attention" and m.get("kv_from") is not None:
                j = m["kv_from"]
                if not (isinstance(j, int) and 0 <= j < i and layers[j].get("type") == "attention"
                        and (layers[j].get("mixer") or {}).get("kv_from") is None):
                    problems.append(f"layer {i}: kv_from must name an earlier attention layer with keys of its own")
            mlp = layer.get("mlp")
            if mlp is not None and (mlp.get("kind", "dense") != "dense" or mlp.get("ff") is None):
                problems.append(f"layer {i}: the feed-forward must be {{'kind': 'dense', 'ff': n}} or null")
            rank = None
            if kind == "channel_delta":
                a1, g1 = (shapes or {}).get(f"l{i}.mix.a1"), (shapes or {}).get(f"l{i}.mix.g1")
                if a1 is not None and g1 is not None:
                    rank = (int(a1[0]), int(g1[0]))
                elif m.get("rank") is not None:
                    rank = (int(m["rank"]), int(m["rank"]))
                else:
                    problems.append(f"layer {i}: the low ranks are given neither by checkpoint tensors "
                                    f"(l{i}.mix.a1, l{i}.mix.g1) nor by the mixer key 'rank'")
            ranks.append(rank)
        # A layer without feed-forward has no second sublayer.  If a checkpoint holds a second norm for
        # such a layer all the same, the norm is applied to alpha * x alone.
        bare = tuple(i for i, layer in enumerate(layers)
                     if layer.get("mlp") is None and f"l{i}.norm2" in (shapes or {}))
        if problems:
            raise ValueError("Bavutar config.json cannot be used: " + "; ".join(problems))
        cap = raw.get("logit_softcap")
        return cls(vocab=int(raw["vocab"]), width=int(raw["width"]), layers=tuple(layers),
                   embedding_scale=float((raw.get("embedding") or {}).get("scale", 1.0)),
                   postln_alpha=float(raw.get("postln_alpha", 1.0)),
                   norm_eps=float((raw.get("norm") or {}).get("eps", 1e-6)),
                   logit_softcap=float(cap) if cap else None,
                   max_position=int(raw.get("max_position", DEFAULT_MAX_POSITION)), ranks=tuple(ranks),
                   bare_second_norm=bare)


def _attention(cfg, i, m, p):
    d, dv, H, G = int(m["dim"]), int(m["vdim"]), int(m["heads"]), int(m["kv_heads"])
    own = m.get("kv_from") is None
    temp = m.get("q_temp")
    spec = AttentionSpec(hidden_size=cfg.width, num_heads=H, num_kv_heads=G, head_dim=d,
                         scale=float(m.get("scale", d ** -0.5)), qk_norm="whole_projection", qk_norm_eps=cfg.norm_eps,
                         prep="general", v_head_dim=None if dv == d else dv,
                         q_temperature=(float(temp["coef"]), int(temp["every"])) if temp else None, own_kv=own)
    qkv = [Source(p + "q", ((0, H * d),))]
    sources = {"mixer.q_norm": (Source(p + "q.norm"),), "mixer.o": (Source(p + "o"),)}
    if own:
        qkv += [Source(p + "k", ((H * d, G * d),)), Source(p + "v", ((H * d + G * d, G * dv),))]
        sources["mixer.k_norm"] = (Source(p + "k.norm"),)
    sources["mixer.qkv"] = tuple(qkv)
    return spec, sources


def _state_space(cfg, i, m, p):
    spec = StateSpaceSpec(hidden_size=cfg.width, num_heads=int(m["heads"]), head_dim=int(m["vdim"]),
                          state_size=int(m["state"]), groups=int(m["groups"]), conv_taps=int(m["conv"]),
                          norm_groups=int(m["norm_groups"]), norm_eps=cfg.norm_eps)
    names = {"in_proj": "in", "conv_w": "conv", "conv_b": "conv.b", "dt_bias": "dt_bias", "a_log": "A_log",
             "d_skip": "D", "norm_w": "norm", "o": "o"}
    return spec, {f"mixer.{k}": (Source(p + v),) for k, v in names.items()}


def _gated_delta(cfg, i, m, p):
    d, dv, H, G = int(m["dim"]), int(m["vdim"]), int(m["heads"]), int(m["kv_heads"])
    ra, rg = cfg.ranks[i]
    spec = GatedDeltaSpec(hidden_size=cfg.width, num_heads=H, num_kv_heads=G, head_dim=d, v_head_dim=dv,
                          conv_taps=int(m["conv"]), decay_rank=ra, gate_rank=rg, norm_eps=cfg.norm_eps)
    qk, vv = G * d, H * dv
    rows, at = [], 0
    for name, n in (("q", qk), ("k", qk), ("v", vv), ("b", H), ("a1", ra), ("g1", rg)):
        rows.append(Source(p + name, ((at, n),)))
        at += n
    conv = (Source(p + "q.conv", ((0, qk),)), Source(p + "k.conv", ((qk, qk),)), Source(p + "v.conv", ((2 * qk, vv),)))
    sources = {"mixer.in_proj": tuple(rows), "mixer.conv_w": conv, "mixer.a2": (Source(p + "a2"),),
               "mixer.g2": (Source(p + "g2"),), "mixer.dt_bias": (Source(p + "dt_bias"),),
               "mixer.a_log": (Source(p + "A_log"),), "mixer.norm_w": (Source(p + "norm"),), "mixer.o": (Source(p + "o"),)}
    return spec, sources


_MIXERS = {"attention": _attention, "mamba2": _state_space, "channel_delta": _gated_delta}


def build_bavutar(cfg: BavutarConfig) -> ModelSpec:
    norm = LayerNormSpec(size=cfg.width, eps=cfg.norm_eps, bias=True)
    layers, order = [], []
    for i, layer in enumerate(cfg.layers):
        m = layer["mixer"]
        mixer, sources = _MIXERS[layer["type"]](cfg, i, m, f"l{i}.mix.")
        sources["mixer_norm.weight"] = (Source(f"l{i}.norm1"),)
        sources["mixer_norm.bias"] = (Source(f"l{i}.norm1.b"),)
        ff = None
        if layer.get("mlp") is not None:
            ff = PlainMLPSpec(hidden_size=cfg.width, intermediate_size=int(layer["mlp"]["ff"]), activation="relu2")
            sources["feed_forward.up"] = (Source(f"l{i}.mlp.up"),)
            sources["feed_forward.down"] = (Source(f"l{i}.mlp.down"),)
            sources["feed_forward_norm.weight"] = (Source(f"l{i}.norm2"),)
            sources["feed_forward_norm.bias"] = (Source(f"l{i}.norm2.b"),)
        second_norm = ff is not None or i in cfg.bare_second_norm
        if ff is None and second_norm:
            sources["feed_forward_norm.weight"] = (Source(f"l{i}.norm2"),)
            sources["feed_forward_norm.bias"] = (Source(f"l{i}.norm2.b"),)
        layers.append(LayerSpec(mixer=mixer, feed_forward=ff, mixer_norm=norm,
                                feed_forward_norm=norm if second_norm else None, arrangement="post_norm",
                                residual_scale=cfg.postln_alpha, sources=sources))
        shared = m.get("kv_from") if layer["type"] == "attention" else None
        order.append(ScheduleEntry(layer=i, cache=shared, write_cache=shared is None))
    return ModelSpec(architecture=ARCHITECTURE, hidden_size=cfg.width, vocab_size=cfg.vocab,
                     max_position=cfg.max_position, layers=layers, order=order, final_norm=norm,
                     final_norm_sources={"weight": "final.norm", "bias": "final.norm.b"}, embed_source="embed",
                     head_source="head", embed_scale=cfg.embedding_scale, logit_softcap=cfg.logit_softcap,
                     residual_stream="float32")


register_architecture(ARCHITECTURE, BavutarConfig, build_bavutar)
