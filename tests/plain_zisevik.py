"""A plain, slow implementation of the Zisevik design: one function per mechanism, 64-bit torch on
the CPU, whole sequences at once (the recurrence token by token).  It shares no code with the
engine; the tests compare the engine with it.

``config`` is the config.json dictionary, ``w`` maps checkpoint tensor names to tensors.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, weight, eps):
    return unit_rms(x, eps) * weight


def rotate_half_pairs(x, positions, dims, base):
    """x [T, H, D]: dim i of the first ``dims`` is paired with dim i + dims/2; the rest pass."""
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    ang = positions.to(F64)[:, None] * freq[None, :]           # [T, half]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], -1)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def latent_attention(h, w, p, m, eps):
    """h [T, width]; tensors ``p + name``; ``m`` the mixer's configuration."""
    T = h.shape[0]
    H, d, r, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    cq = rms_norm(h @ w[p + "dq"].T, w[p + "dq.norm"], eps)
    q = (cq @ w[p + "uq"].T).view(T, H, d + r)
    q_plain, q_rot = q[..., :d], rotate_half_pairs(q[..., d:], pos, m["rot"]["dims"], m["rot"]["base"])
    kv = h @ w[p + "dkv"].T
    c = rms_norm(kv[:, :rank], w[p + "dkv.norm"], eps)
    k_rot = rotate_half_pairs(kv[:, None, rank:], pos, m["rot"]["dims"], m["rot"]["base"])[:, 0]    # [T, r], all heads
    k_plain = (c @ w[p + "uk"].T).view(T, H, d)
    v = (c @ w[p + "uv"].T).view(T, H, dv)
    scores = (torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihd,jd->hij", q_rot, k_rot)) * m["scale"]
    i, j = pos[:, None], pos[None, :]
    seen = i - j >= 0
    if m.get("mask"):                                             # a sliding window; without one every earlier key is seen
        seen = seen & (i - j < m["mask"]["size"])
    scores = scores.masked_fill(~seen[None], float("-inf"))
    sink = w[p + "sink"].to(F64)[:, None, None].expand(H, T, 1)
    both = torch.cat([scores, sink], -1)
    prob = torch.softmax(both, -1)[..., :T]                      # the sink has no value
    out = torch.einsum("hij,jhd->ihd", prob, v).reshape(T, H * dv)
    return out @ w[p + "o"].T


def retention(h, w, p, m, eps):
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = rotate_half_pairs((h @ w[p + "q"].T).view(T, H, d), pos, m["rot"]["dims"], m["rot"]["base"])
    k = rotate_half_pairs((h @ w[p + "k"].T).view(T, H, d), pos, m["rot"]["dims"], m["rot"]["base"]) * d ** -0.5
    v = (h @ w[p + "v"].T).view(T, H, dv)
    decay = torch.tensor(m["decay"], dtype=F64)
    S = torch.zeros(H, d, dv, dtype=F64)
    o = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = unit_rms(o, eps).reshape(T, H * dv)
    return (o * silu(h @ w[p + "g"].T)) @ w[p + "o"].T


def dense_ff(h, w, p):
    return gelu_tanh(h @ w[p + "up"].T) @ w[p + "down"].T


def moe_ff(h, w, p, mlp):
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    z = h @ w[p + "router"].T + w[p + "router.b"]
    val, idx = torch.topk(z, top, dim=-1)
    share = torch.softmax(val, -1)
    out = torch.zeros_like(h)
    for e in range(E):
        y = (silu(h @ w[p + f"e{e}.gate"].T) * (h @ w[p + f"e{e}.up"].T)) @ w[p + f"e{e}.down"].T
        weight = (share * (idx == e)).sum(-1, keepdim=True)
        out = out + weight * y
    return out


MIXERS = {"latent_attention": latent_attention, "retention": retention}


def layer(x, w, i, spec, eps):
    p = f"l{i}."
    x = x + MIXERS[spec["type"]](rms_norm(x, w[p + "norm1"], eps), w, p + "mix.", spec["mixer"], eps)
    mlp = spec.get("mlp")
    if mlp is not None:
        hn = rms_norm(x, w[p + "norm2"], eps)
        x = x + (dense_ff(hn, w, p + "mlp.") if mlp["kind"] == "dense" else moe_ff(hn, w, p + "mlp.", mlp))
    return x


def layer_runs(config):
    """The layers in the order they run, as (layer index, starts a pass)."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    runs = [(i, False) for i in range(a)]
    for _ in range(times):
        runs += [(i, i == a) for i in range(a, b)]
    return runs + [(i, False) for i in range(b, n)]


def forward(config, weights, tokens, taps=None):
    """Logits [T, vocab] of one sequence (64-bit).  ``taps``: a list that receives the stream after
    every layer run."""
    w = {k: (v.to(F64) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = config["norm"]["eps"]
    x0 = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    x = x0
    for i, first in layer_runs(config):
        if first:
            x = torch.cat([x, x0], -1) @ w["loop.in"].T
        x = layer(x, w, i, config["layers"][i], eps)
        if taps is not None:
            taps.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T


def tensor_shapes(config):
    """Checkpoint tensor name -> shape, for a configuration dictionary."""
    W = config["width"]
    out = {"embed": (config["vocab"], W), "head": (config["vocab"], W), "final.norm": (W,)}
    if config.get("loop"):
        out["loop.in"] = (W, 2 * W)
    for i, spec in enumerate(config["layers"]):
        p, m = f"l{i}.", spec["mixer"]
        out[p + "norm1"] = (W,)
        H, d, dv = m["heads"], m["dim"], m["vdim"]
        if spec["type"] == "retention":
            out.update({p + "mix.q": (H * d, W), p + "mix.k": (H * d, W), p + "mix.v": (H * dv, W),
                        p + "mix.g": (H * dv, W), p + "mix.o": (W, H * dv)})
        else:
            r, qr, kr = m["rot_dim"], m["q_rank"], m["kv_rank"]
            out.update({p + "mix.dq": (qr, W), p + "mix.dq.norm": (qr,), p + "mix.uq": (H * (d + r), qr),
                        p + "mix.dkv": (kr + r, W), p + "mix.dkv.norm": (kr,), p + "mix.uk": (H * d, kr),
                        p + "mix.uv": (H * dv, kr), p + "mix.sink": (H,), p + "mix.o": (W, H * dv)})
        mlp = spec.get("mlp")
        if mlp is None:
            continue
        out[p + "norm2"] = (W,)
        if mlp["kind"] == "dense":
            out.update({p + "mlp.up": (mlp["ff"], W), p + "mlp.down": (W, mlp["ff"])})
        else:
            E, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
            out.update({p + "mlp.router": (E, W), p + "mlp.router.b": (E,)})
            for e in range(E):
                out.update({p + f"mlp.e{e}.gate": (ff, W), p + f"mlp.e{e}.up": (ff, W), p + f"mlp.e{e}.down": (W, ff)})
    return out


def random_weights(config, seed, gain=1.0):
    """bfloat16 tensors of a size that keeps activations of order one."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(config).items():
        x = torch.randn(shape, generator=g)
        if name.endswith(("norm", "norm1", "norm2")):
            t = 1.0 + 0.2 * x
        elif name.endswith(("sink", "router.b")):
            t = 0.7 * x
        elif name == "embed":
            t = x
        else:
            t = gain * x / math.sqrt(shape[-1])
        out[name] = t.to(torch.bfloat16)
    return out
