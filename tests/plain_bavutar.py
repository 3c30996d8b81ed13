"""A plain, slow implementation of the Bavutar design: one function per mechanism, whole
sequences at a time, token-by-token loops for everything recurrent, torch on the CPU in one
floating type (32- or 64-bit).  It shares no code with the engine; the GPU tests compare the
engine with it.

Notation: ``h`` [T, width] is a sublayer's input, ``W`` matrices are stored [out, in] and
applied as ``h @ W.T``; a layer's tensors are looked up as ``w[prefix + name]``.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def layer_norm(x, weight, bias, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * weight + bias


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def causal_conv(x, taps_w, bias=None):
    """x [T, C]; taps_w [C, taps], the last column multiplies the current token; zeros before
    the sequence."""
    T, C = x.shape
    taps = taps_w.shape[1]
    pad = torch.cat([x.new_zeros(taps - 1, C), x], 0)
    out = x.new_zeros(T, C)
    for j in range(taps):
        out = out + pad[j:j + T] * taps_w[:, j]
    if bias is not None:
        out = out + bias
    return out


def query_temperature(positions, coef, every):
    """1 + coef * ln(floor((p + 1) / every) + 1) for every position."""
    steps = torch.div(positions + 1, every, rounding_mode="floor")
    return 1.0 + coef * torch.log(steps.to(torch.float64) + 1.0)


def attention_keys_values(h, w, p, m, eps):
    """The keys (after their norm) and values a layer keeps: [T, G, dim], [T, G, vdim]."""
    T = h.shape[0]
    k = rms(h @ w[p + "k"].T, eps) * w[p + "k.norm"]
    v = h @ w[p + "v"].T
    return k.view(T, m["kv_heads"], m["dim"]), v.view(T, m["kv_heads"], m["vdim"])


def attention(h, w, p, m, eps, keys, values):
    """Softmax attention of this layer's queries over the given keys and values (its own, or
    those of the layer it borrows them from)."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms(h @ w[p + "q"].T, eps) * w[p + "q.norm"]
    pos = torch.arange(T)
    if m.get("q_temp"):
        q = q * query_temperature(pos, m["q_temp"]["coef"], m["q_temp"]["every"]).to(q.dtype)[:, None]
    q = q.view(T, H, d)
    scale = m.get("scale", d ** -0.5)
    out = h.new_zeros(T, H, dv)
    mask = pos[None, :] <= pos[:, None]
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ keys[:, g].T) * scale
        s = s.masked_fill(~mask, float("-inf"))
        out[:, head] = torch.softmax(s, -1) @ values[:, g]
    return out.reshape(T, H * dv) @ w[p + "o"].T


def mamba2(h, w, p, m, eps):
    T = h.shape[0]
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    proj = h @ w[p + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = F.silu(causal_conv(xbc, w[p + "conv"], w[p + "conv.b"]))
    x = xbc[:, :inner].view(T, H, P)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    dt = F.softplus(dt + w[p + "dt_bias"])
    rate = torch.exp(w[p + "A_log"])
    y = h.new_zeros(T, H, P)
    for head in range(H):
        g = head // (H // G)
        S = h.new_zeros(N, P)
        for t in range(T):
            S = torch.exp(-rate[head] * dt[t, head]) * S + dt[t, head] * torch.outer(B[t, g], x[t, head])
            y[t, head] = S.T @ C[t, g] + w[p + "D"][head] * x[t, head]
    y = y.reshape(T, inner) * F.silu(z)
    parts = m["norm_groups"]
    y = rms(y.view(T, parts, inner // parts), eps).reshape(T, inner) * w[p + "norm"]
    return y @ w[p + "o"].T


def channel_delta(h, w, p, m, eps):
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = F.silu(causal_conv(h @ w[p + "q"].T, w[p + "q.conv"])).view(T, G, d)
    k = F.silu(causal_conv(h @ w[p + "k"].T, w[p + "k.conv"])).view(T, G, d)
    v = F.silu(causal_conv(h @ w[p + "v"].T, w[p + "v.conv"])).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[p + "b"].T)                                   # [T, H]
    a = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "dt_bias"]
    decay = torch.exp(-torch.exp(w[p + "A_log"])[None, :, None] * F.softplus(a).view(T, H, d))
    gate = torch.sigmoid((h @ w[p + "g1"].T) @ w[p + "g2"].T).view(T, H, dv)
    o = h.new_zeros(T, H, dv)
    for head in range(H):
        g = head // (H // G)
        S = h.new_zeros(d, dv)
        for t in range(T):
            S = decay[t, head][:, None] * S
            u = beta[t, head] * (v[t, head] - S.T @ k[t, g])
            S = S + torch.outer(k[t, g], u)
            o[t, head] = S.T @ q[t, g]
    o = rms(o, eps) * w[p + "norm"] * gate
    return o.reshape(T, H * dv) @ w[p + "o"].T


def feed_forward(h, w, p):
    return (torch.relu(h @ w[p + "up"].T) ** 2) @ w[p + "down"].T


def forward(config, weights, tokens, dtype=torch.float64, layers_out=None):
    """Logits [T, vocab] of one sequence.  ``layers_out``: a list that receives the residual
    stream after every layer."""
    w = {k: v.to(dtype) for k, v in weights.items()}
    eps = config["norm"]["eps"]
    alpha = config["postln_alpha"]
    tok = torch.as_tensor(tokens, dtype=torch.long)
    x = w["embed"][tok] * config["embedding"]["scale"]
    kept = {}
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.mix.", layer["mixer"]
        if layer["type"] == "attention":
            src = m.get("kv_from")
            if src is None:
                kept[i] = attention_keys_values(x, w, p, m, eps)
                src = i
            y = attention(x, w, p, m, eps, *kept[src])
        elif layer["type"] == "mamba2":
            y = mamba2(x, w, p, m, eps)
        elif layer["type"] == "channel_delta":
            y = channel_delta(x, w, p, m, eps)
        else:
            raise ValueError(layer["type"])
        x = layer_norm(alpha * x + y, w[f"l{i}.norm1"], w[f"l{i}.norm1.b"], eps)
        if layer.get("mlp"):
            x = layer_norm(alpha * x + feed_forward(x, w, f"l{i}.mlp."), w[f"l{i}.norm2"], w[f"l{i}.norm2.b"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    x = layer_norm(x, w["final.norm"], w["final.norm.b"], eps)
    logits = x @ w["head"].T
    cap = config.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return logits


def tensor_shapes(config):
    """Name -> shape of every checkpoint tensor of a configuration."""
    W, out = config["width"], {}
    out["embed"] = (config["vocab"], W)
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.mix.", layer["mixer"]
        out[f"l{i}.norm1"] = out[f"l{i}.norm1.b"] = (W,)
        if layer["type"] == "attention":
            out[p + "q"] = (m["heads"] * m["dim"], W)
            out[p + "q.norm"] = (m["heads"] * m["dim"],)
            if m.get("kv_from") is None:
                out[p + "k"] = (m["kv_heads"] * m["dim"], W)
                out[p + "k.norm"] = (m["kv_heads"] * m["dim"],)
                out[p + "v"] = (m["kv_heads"] * m["vdim"], W)
            out[p + "o"] = (W, m["heads"] * m["vdim"])
        elif layer["type"] == "mamba2":
            inner, gn = m["heads"] * m["vdim"], m["groups"] * m["state"]
            out[p + "in"] = (2 * inner + 2 * gn + m["heads"], W)
            out[p + "conv"] = (inner + 2 * gn, m["conv"])
            out[p + "conv.b"] = (inner + 2 * gn,)
            out[p + "dt_bias"] = out[p + "A_log"] = out[p + "D"] = (m["heads"],)
            out[p + "norm"] = (inner,)
            out[p + "o"] = (W, inner)
        else:
            qk, vv, r = m["kv_heads"] * m["dim"], m["heads"] * m["vdim"], m.get("rank", 8)
            out[p + "q"], out[p + "k"], out[p + "v"] = (qk, W), (qk, W), (vv, W)
            out[p + "q.conv"], out[p + "k.conv"], out[p + "v.conv"] = (qk, m["conv"]), (qk, m["conv"]), (vv, m["conv"])
            out[p + "b"] = (m["heads"], W)
            out[p + "A_log"] = (m["heads"],)
            out[p + "norm"] = (m["vdim"],)
            out[p + "a1"], out[p + "a2"] = (r, W), (m["heads"] * m["dim"], r)
            out[p + "dt_bias"] = (m["heads"] * m["dim"],)
            out[p + "g1"], out[p + "g2"] = (r, W), (vv, r)
            out[p + "o"] = (W, vv)
        if layer.get("mlp"):
            out[f"l{i}.norm2"] = out[f"l{i}.norm2.b"] = (W,)
            out[f"l{i}.mlp.up"] = (layer["mlp"]["ff"], W)
            out[f"l{i}.mlp.down"] = (W, layer["mlp"]["ff"])
    out["final.norm"] = out["final.norm.b"] = (W,)
    out["head"] = (config["vocab"], W)
    return out


def random_weights(config, seed, *, std=None):
    """Random weights that keep every mechanism visible: matrices N(0, 1/sqrt(in)), norm
    weights around 1, small biases, decays spread over (0, 1)."""
    g = torch.Generator().manual_seed(seed)
    w = {}
    for name, shape in tensor_shapes(config).items():
        last = name.rsplit(".", 1)[-1]
        if len(shape) == 2 and not name.endswith(".conv"):
            s = std if std is not None else 1.0 / math.sqrt(shape[1])
            w[name] = torch.randn(shape, generator=g) * s
        elif name.endswith(".conv"):
            w[name] = torch.randn(shape, generator=g) * 0.5
        elif last in ("norm1", "norm2", "norm") or name == "final.norm":
            w[name] = 1.0 + 0.1 * torch.randn(shape, generator=g)
        elif last == "A_log":
            w[name] = torch.randn(shape, generator=g) * 0.5 - 0.5
        elif last == "D":
            w[name] = 1.0 + 0.2 * torch.randn(shape, generator=g)
        else:       # biases
            w[name] = 0.1 * torch.randn(shape, generator=g)
    return {k: v.to(torch.bfloat16) for k, v in w.items()}
