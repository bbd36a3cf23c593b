"""A plain, slow Sitelorn: every mechanism as one function over whole sequences, float64 on the CPU.

It shares nothing with the engine: no kernels, no cache, no batching.  A sequence is run whole, token after token
where a mechanism is a recurrence, so that the engine's portions, batches, pages and state slots have something to be
held against.  ``tensors`` maps checkpoint names to torch tensors; ``cfg`` is the dict of a config.json.

Notation: T tokens, D the model's width, H heads, G key/value heads, dk / dv the size of a key / value head.
"""
from __future__ import annotations

import math

import torch

F = torch.float64


def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def layer_norm(x, w, b, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def linear_recurrence(q, k, v, decay):
    """S_t = diag(decay_t) S_(t-1) + k_t v_t^T,  o_t = S_t^T q_t.

    q, k: [T, H, dk]; v: [T, H, dv]; decay: [T, H, dk] (a per-head constant is given as such a tensor too).
    Returns o [T, H, dv]."""
    T, H, dk = q.shape
    dv = v.shape[-1]
    S = torch.zeros(H, dk, dv, dtype=F)
    out = torch.zeros(T, H, dv, dtype=F)
    for t in range(T):
        S = decay[t].unsqueeze(-1) * S + k[t].unsqueeze(-1) * v[t].unsqueeze(-2)
        out[t] = torch.einsum("hkv,hk->hv", S, q[t])
    return out


def lightning_mixer(h, m, W, prefix, eps):
    """Linear attention with one constant decay per head; silu on q, k, v; one RMS norm over all heads; sigmoid gate."""
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ W[prefix + "q"].T).view(T, H, dk)
    k = silu(h @ W[prefix + "k"].T).view(T, H, dk)
    v = silu(h @ W[prefix + "v"].T).view(T, H, dv)
    decay = torch.tensor(m["decay"], dtype=F).view(1, H, 1).expand(T, H, dk)
    o = linear_recurrence(q, k, v, decay).reshape(T, H * dv)
    o = rms(o, eps) * W[prefix + "norm"]
    o = o * torch.sigmoid(h @ W[prefix + "g"].T)
    return o @ W[prefix + "o"].T


def gla_mixer(h, m, W, prefix, eps):
    """Linear attention with a decay per key channel and token, made by a two-step projection; per-head RMS norm over
    the value size with one shared weight; silu gate."""
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ W[prefix + "q"].T).view(T, H, dk) * dk ** -0.5
    k = (h @ W[prefix + "k"].T).view(T, H, dk)
    v = (h @ W[prefix + "v"].T).view(T, H, dv)
    z = (h @ W[prefix + "a1"].T) @ W[prefix + "a2"].T + W[prefix + "a2.b"]
    alpha = torch.exp(torch.nn.functional.logsigmoid(z) / m["tau"]).view(T, H, dk)
    o = linear_recurrence(q, k, v, alpha)
    o = rms(o, eps) * W[prefix + "norm"]
    o = o.reshape(T, H * dv) * silu(h @ W[prefix + "g"].T)
    return o @ W[prefix + "o"].T


def short_conv(u, w):
    """y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the start.  u [T, C], w [C, taps]."""
    T, C = u.shape
    taps = w.shape[1]
    pad = torch.cat([torch.zeros(taps - 1, C, dtype=F), u], 0)
    y = torch.zeros(T, C, dtype=F)
    for j in range(taps):
        y = y + w[:, j] * pad[j: j + T]
    return y


def rotate_pairs(x, rot):
    """Rotate the pairs (2i, 2i+1), i < dims/2, of every head by position * base^(-2i/dims).  x [T, H, d]."""
    dims, base = rot["dims"], rot["base"]
    T = x.shape[0]
    i = torch.arange(dims // 2, dtype=F)
    ang = torch.arange(T, dtype=F).view(T, 1) * base ** (-2.0 * i / dims)
    c, s = torch.cos(ang).view(T, 1, -1), torch.sin(ang).view(T, 1, -1)
    out = x.clone()
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def attention_keys_values(h, m, W, prefix, eps):
    """The keys (after convolution, norm over the whole projection, rotation) and values (after convolution)."""
    T = h.shape[0]
    G, dk, dv = m["kv_heads"], m["dim"], m["vdim"]
    k = short_conv(h @ W[prefix + "k"].T, W[prefix + "k.conv"])
    v = short_conv(h @ W[prefix + "v"].T, W[prefix + "v.conv"])
    k = rms(k, eps) * W[prefix + "k.norm"]
    return rotate_pairs(k.view(T, G, dk), m["rot"]), v.view(T, G, dv)


def windowed_sink_attention(q, k, v, scale, window):
    """p_j = exp(s_j) / (1 + sum exp(s_j)) over the keys j with 0 <= i - j < window.  q [T, H, dk], k [T, G, dk]."""
    T, H, dk = q.shape
    G = k.shape[1]
    rep = H // G
    out = torch.zeros(T, H, v.shape[-1], dtype=F)
    i = torch.arange(T).view(T, 1)
    j = torch.arange(T).view(1, T)
    seen = (i - j >= 0) & (i - j < window)
    for hd in range(H):
        g = hd // rep
        s = (q[:, hd] @ k[:, g].T) * scale
        s = s.masked_fill(~seen, -math.inf)
        mx = torch.clamp(s.max(-1, keepdim=True).values, min=0.0)
        e = torch.exp(s - mx)
        p = e / (torch.exp(-mx) + e.sum(-1, keepdim=True))
        out[:, hd] = p @ v[:, g]
    return out


def attention_mixer(h, m, W, prefix, eps, kv):
    """``kv``: (keys, values) of the layer this one borrows from, or None to make its own."""
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = short_conv(h @ W[prefix + "q"].T, W[prefix + "q.conv"])
    q = rotate_pairs((rms(q, eps) * W[prefix + "q.norm"]).view(T, H, dk), m["rot"])
    if kv is None:
        kv = attention_keys_values(h, m, W, prefix, eps)
    o = windowed_sink_attention(q, kv[0], kv[1], m["scale"], m["mask"]["size"])
    o = o * torch.sigmoid(h @ W[prefix + "g"].T).view(T, H, 1)
    return o.reshape(T, H * dv) @ W[prefix + "o"].T, kv


def feed_forward(h, W, prefix):
    return (gelu_tanh(h @ W[prefix + "gate"].T) * (h @ W[prefix + "up"].T)) @ W[prefix + "down"].T


def forward(cfg, tensors, tokens, return_layers=False):
    """Logits [T, vocab] of one whole sequence (and the stream after every layer)."""
    W = {n: t.to(F) for n, t in tensors.items() if t.dtype.is_floating_point}
    eps = cfg["norm"]["eps"]
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)] * cfg["embedding"]["scale"]
    kvs = {}
    layers = []
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        if layer["type"] == "lightning":
            y = lightning_mixer(x, m, W, p + "mix.", eps)
        elif layer["type"] == "gla":
            y = gla_mixer(x, m, W, p + "mix.", eps)
        elif layer["type"] == "attention":
            src = m.get("kv_from")
            y, kvs[i] = attention_mixer(x, m, W, p + "mix.", eps, None if src is None else kvs[src])
        else:
            raise ValueError(layer["type"])
        x = x + layer_norm(y, W[p + "norm1"], W[p + "norm1.b"], eps)
        if layer.get("mlp") is not None:
            x = x + layer_norm(feed_forward(x, W, p + "mlp."), W[p + "norm2"], W[p + "norm2.b"], eps)
        layers.append(x)
    logits = layer_norm(x, W["final.norm"], W["final.norm.b"], eps) @ W["head"].T
    return (logits, torch.stack(layers)) if return_layers else logits
