"""Zisevik: a decoder-only design whose ``config.json`` lists its layers one by one, some of which
run several times in a row.

Every layer is pre-norm over a 32-bit stream: ``x <- x + mixer(norm1(x))`` and, where the layer has a
feed-forward, ``x <- x + ff(norm2(x))``, with RMS norms.  A layer's mixer is one of

* ``latent_attention``: softmax attention over a cached latent (``parts.latent_attention``): queries
  through a normed latent, one normed key/value latent per position plus a rotated key part shared
  by the heads, a sliding window, and a learned sink logit per head in the softmax's denominator;
* ``retention``: linear attention with a fixed decay per head (``parts.recurrent.RetentionMixer``).

The feed-forward is ``dense`` (ungated, tanh-form gelu) or ``moe`` (SwiGLU experts; the router's bias
is part of its logits, the largest logits are chosen and weighed by a softmax among themselves).
``loop``: layers ``start .. stop-1`` run ``times`` times in a row with the same weights, each pass
with a cache or state of its own; before the first layer of every pass the stream becomes
``W_in [x; x0]`` with ``x0`` the embedding output.  The final norm is an RMS norm.

Tensor names: ``embed``, ``head``, ``final.norm``, ``loop.in``, ``l<i>.norm1|norm2``, ``l<i>.mix.*``,
``l<i>.mlp.up|down`` or ``l<i>.mlp.router[.b]`` and ``l<i>.mlp.e<j>.gate|up|down``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from ..config.registry import register_architecture
from ..config.specs import (LatentAttentionSpec, LayerSpec, ModelSpec, MoESpec, PlainMLPSpec, RetentionSpec,
                            RMSNormSpec, RotarySpec, ScheduleEntry, Source)

ARCHITECTURE = "Zisevik"
MIXER_TYPES = ("latent_attention", "retention")
DEFAULT_MAX_POSITION = 1 << 20      # the design has no position table; the cache manager wants a bound

_MIXER_KEYS = {"latent_attention": ("heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank"),
               "retention": ("heads", "dim", "vdim", "decay")}


@dataclass(frozen=True)
class ZisevikConfig:
    vocab: int
    width: int
    layers: tuple                      # of dicts {"type", "mixer", "mlp"} as in config.json (validated)
    loop: Optional[tuple]              # (start, stop, times) or None
    norm_eps: float
    max_position: int

    @classmethod
    def from_dict(cls, raw: dict) -> "ZisevikConfig":
        problems = []
        for key in ("vocab", "width", "layers"):
            if raw.get(key) is None:
                problems.append(f"missing key {key!r}")
        layers = raw.get("layers") or []
        if not isinstance(layers, list) or not layers:
            problems.append("'layers' must be a non-empty list")
            layers = []
        for i, layer in enumerate(layers):
            kind, m = layer.get("type"), layer.get("mixer") or {}
            if kind not in MIXER_TYPES:
                problems.append(f"layer {i}: unknown mixer type {kind!r} (known: {', '.join(MIXER_TYPES)})")
                continue
            missing = [k for k in _MIXER_KEYS[kind] if m.get(k) is None]
            if missing:
                problems.append(f"layer {i} ({kind}): missing mixer keys {missing}")
            rot = m.get("rot")
            if rot is not None and (rot.get("dims") is None or rot.get("base") is None):
                problems.append(f"layer {i}: 'rot' needs 'dims' and 'base'")
            if kind == "retention" and m.get("decay") is not None and len(m["decay"]) != m.get("heads"):
                problems.append(f"layer {i}: 'decay' needs one entry per head")
            mlp = layer.get("mlp")
            if mlp is not None:
                if mlp.get("kind") == "dense":
                    if mlp.get("ff") is None:
                        problems.append(f"layer {i}: a dense feed-forward needs 'ff'")
                elif mlp.get("kind") == "moe":
                    if (mlp.get("expert") or {}).get("ff") is None or (mlp.get("router") or {}).get("experts") is None \
                            or (mlp.get("router") or {}).get("top") is None:
                        problems.append(f"layer {i}: a moe feed-forward needs expert.ff, router.experts and router.top")
                else:
                    problems.append(f"layer {i}: the feed-forward's kind must be 'dense' or 'moe', or the entry null")
        loop = raw.get("loop")
        if loop is not None:
            try:
                loop = (int(loop["start"]), int(loop["stop"]), int(loop["times"]))
                if not (0 <= loop[0] < loop[1] <= len(layers) and loop[2] >= 1):
                    problems.append(f"loop {loop} does not fit {len(layers)} layers")
            except (KeyError, TypeError, ValueError):
                problems.append("'loop' needs integer 'start', 'stop' and 'times'")
        if problems:
            raise ValueError("Zisevik config.json cannot be used: " + "; ".join(problems))
        return cls(vocab=int(raw["vocab"]), width=int(raw["width"]), layers=tuple(layers), loop=loop,
                   norm_eps=float((raw.get("norm") or {}).get("eps", 1e-6)),
                   max_position=int(raw.get("max_position", DEFAULT_MAX_POSITION)))


def _rotary(m, default_dims):
    rot = m.get("rot")
    if rot is None or int(rot["dims"]) == 0:
        return None
    return RotarySpec(rotary_dim=int(rot["dims"]), theta=float(rot["base"]), pairing="split_half")


def _latent_attention(cfg, m, p):
    H, d, r, dv = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"])
    q_rank, rank = int(m["q_rank"]), int(m["kv_rank"])
    window = (m.get("mask") or {}).get("size")
    spec = LatentAttentionSpec(hidden_size=cfg.width, num_heads=H, head_dim=d, rot_dim=r, v_head_dim=dv, q_rank=q_rank,
                               kv_rank=rank, scale=float(m.get("scale", (d + r) ** -0.5)), window=int(window) if window else None, sink=True,
                               position=_rotary(m, r), norm_eps=cfg.norm_eps)
    sources = {"mixer.down": (Source(p + "dq", ((0, q_rank),)), Source(p + "dkv", ((q_rank, rank + r),))),
               "mixer.q_norm": (Source(p + "dq.norm"),), "mixer.kv_norm": (Source(p + "dkv.norm"),),
               "mixer.uq": (Source(p + "uq"),), "mixer.uk": (Source(p + "uk"),), "mixer.uv": (Source(p + "uv"),),
               "mixer.sink": (Source(p + "sink"),), "mixer.o": (Source(p + "o"),)}
    return spec, sources


def _retention(cfg, m, p):
    H, d, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    spec = RetentionSpec(hidden_size=cfg.width, num_heads=H, head_dim=d, v_head_dim=dv,
                         decays=tuple(float(g) for g in m["decay"]), position=_rotary(m, d), norm_eps=cfg.norm_eps)
    rows, at = [], 0
    for name, n in (("q", H * d), ("k", H * d), ("v", H * dv), ("g", H * dv)):
        rows.append(Source(p + name, ((at, n),)))
        at += n
    return spec, {"mixer.in_proj": tuple(rows), "mixer.o": (Source(p + "o"),)}


_MIXERS = {"latent_attention": _latent_attention, "retention": _retention}


def _feed_forward(cfg, mlp, p):
    if mlp["kind"] == "dense":
        spec = PlainMLPSpec(hidden_size=cfg.width, intermediate_size=int(mlp["ff"]), activation="gelu_tanh")
        return spec, {"feed_forward.up": (Source(p + "up"),), "feed_forward.down": (Source(p + "down"),)}
    E, top, ff = int(mlp["router"]["experts"]), int(mlp["router"]["top"]), int(mlp["expert"]["ff"])
    spec = MoESpec(hidden_size=cfg.width, num_experts=E, top_k=top, intermediate_size=ff, score_fn="top_softmax",
                   selection_bias=True, renormalize=True, routed_scale=1.0, activation="silu")
    w13, w2 = [], []
    for e in range(E):
        w13 += [Source(p + f"e{e}.gate", (e, (0, ff))), Source(p + f"e{e}.up", (e, (ff, ff)))]
        w2.append(Source(p + f"e{e}.down", (e,)))
    return spec, {"feed_forward.gate": (Source(p + "router"),), "feed_forward.selection_bias": (Source(p + "router.b"),),
                  "feed_forward.w13": tuple(w13), "feed_forward.w2": tuple(w2)}


def layer_order(num_layers: int, loop) -> list:
    """The visits in the order they run: ``(layer, starts a pass)``."""
    if loop is None:
        return [(i, False) for i in range(num_layers)]
    start, stop, times = loop
    runs = [(i, False) for i in range(start)]
    for _ in range(times):
        runs += [(i, i == start) for i in range(start, stop)]
    return runs + [(i, False) for i in range(stop, num_layers)]


def build_zisevik(cfg: ZisevikConfig) -> ModelSpec:
    norm = RMSNormSpec(size=cfg.width, eps=cfg.norm_eps)
    layers = []
    for i, layer in enumerate(cfg.layers):
        mixer, sources = _MIXERS[layer["type"]](cfg, layer["mixer"], f"l{i}.mix.")
        sources["mixer_norm.weight"] = (Source(f"l{i}.norm1"),)
        ff = None
        if layer.get("mlp") is not None:
            ff, more = _feed_forward(cfg, layer["mlp"], f"l{i}.mlp.")
            sources.update(more)
            sources["feed_forward_norm.weight"] = (Source(f"l{i}.norm2"),)
        layers.append(LayerSpec(mixer=mixer, feed_forward=ff, mixer_norm=norm,
                                feed_forward_norm=norm if ff is not None else None, arrangement="pre_norm_stream",
                                sources=sources))
    # every visit has a cache or state of its own, also a layer's second and third pass
    order = [ScheduleEntry(layer=i, reinject=first) for i, first in layer_order(len(layers), cfg.loop)]
    return ModelSpec(architecture=ARCHITECTURE, hidden_size=cfg.width, vocab_size=cfg.vocab,
                     max_position=cfg.max_position, layers=layers, order=order, final_norm=norm,
                     final_norm_source="final.norm", embed_source="embed", head_source="head",
                     residual_stream="float32", reinject_source="loop.in" if cfg.loop is not None else None)


register_architecture(ARCHITECTURE, ZisevikConfig, build_zisevik)
