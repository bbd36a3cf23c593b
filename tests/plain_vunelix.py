"""A plain, slow Vunelix: every mechanism as one function over whole sequences, float64 on the CPU.

It shares nothing with the engine: no kernels, no cache, no batching.  A sequence is run whole, token after token
where a mechanism is a recurrence, so that the engine's portions, batches, pages and state slots have something to be
held against.  ``W`` maps checkpoint names to torch tensors; ``cfg`` is the dict of a config.json.

Notation: T tokens, D the model's width, H heads, dn / dr the unrotated / rotated size of a query head, dv the size of
a value head, R the latent size; E inner channels and N states of a selective scan.
"""
from __future__ import annotations

import math

import torch

F = torch.float64


def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def silu(z):
    return z * torch.sigmoid(z)


# ---- rotation ---------------------------------------------------------------------------------------------------
def rotary_frequencies(dims, base, scaling=None):
    """(f [dims / 2], m): pair i turns by p * f_i at position p, and cos and sin are multiplied by m.

    Without ``scaling`` f_i = base ** (-2 i / dims) and m = 1.  With it (factor s, original length L, fast, slow) the
    pairs below ``lo`` keep f_i, those above ``hi`` get f_i / s, those between a mixture, where lo and hi are the pair
    numbers whose wavelength fits ``fast`` and ``slow`` times into L; m = 0.1 ln(s) + 1."""
    i = torch.arange(dims // 2, dtype=F)
    f = float(base) ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    s, L = float(scaling["factor"]), float(scaling["original"])
    where = lambda turns: dims * math.log(L / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(where(float(scaling["fast"]))), 0)
    hi = min(math.ceil(where(float(scaling["slow"]))), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / s * ramp + f * (1.0 - ramp), 0.1 * math.log(s) + 1.0


def rotate_pairs(x, positions, f, m):
    """x [T, ..., n]: elements (2i, 2i+1), i < len(f), turn by positions[t] * f_i; cos and sin times m; the rest
    passes unchanged."""
    n = 2 * f.numel()
    ang = positions.to(F).view(-1, *([1] * (x.dim() - 1))) * f
    c, s = torch.cos(ang) * m, torch.sin(ang) * m
    a, b = x[..., 0:n:2], x[..., 1:n:2]
    out = x.clone()
    out[..., 0:n:2] = a * c - b * s
    out[..., 1:n:2] = b * c + a * s
    return out


# ---- mixers -----------------------------------------------------------------------------------------------------
def latent_attention(h, m, W, p, eps, positions=None):
    """Attention whose keys and values are projections of one small latent vector per token, plus one rotated key part
    that all heads share.  h [T, D] -> [T, D]."""
    T = h.shape[0]
    H, dn, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T) if positions is None else positions
    rot = m["rot"]
    f, mag = rotary_frequencies(int(rot["dims"]), float(rot["base"]), rot.get("scaling"))
    q = (h @ W[p + "q"].T).view(T, H, dn + dr)
    q_plain, q_rot = q[..., :dn], rotate_pairs(q[..., dn:], pos, f, mag)
    down = h @ W[p + "dkv"].T
    latent = rms_norm(down[:, :R], W[p + "dkv.norm"], eps)
    k_rot = rotate_pairs(down[:, R:], pos, f, mag)                       # [T, dr], one for all heads
    k_plain = (latent @ W[p + "uk"].T).view(T, H, dn)
    v = (latent @ W[p + "uv"].T).view(T, H, dv)
    scores = (torch.einsum("thd,shd->hts", q_plain, k_plain) + torch.einsum("thd,sd->hts", q_rot, k_rot)) * float(m["scale"])
    causal = torch.arange(T).view(1, T, 1) >= torch.arange(T).view(1, 1, T)
    weights = torch.softmax(scores.masked_fill(~causal, -math.inf), dim=-1)
    o = torch.einsum("hts,shd->thd", weights, v).reshape(T, H * dv)
    o = o * torch.sigmoid(h @ W[p + "g"].T)
    return o @ W[p + "o"].T


def causal_conv(u, taps, bias):
    """y_t[c] = bias[c] + sum_j taps[c, j] * u_(t - J + 1 + j)[c], zeros before the start; u [T, C], taps [C, J]."""
    T, C = u.shape
    J = taps.shape[1]
    padded = torch.cat([torch.zeros(J - 1, C, dtype=F), u], 0)
    y = bias.expand(T, C).clone()
    for j in range(J):
        y = y + padded[j:j + T] * taps[:, j]
    return y


def selective_scan(x, dt, A, B, C, Dskip):
    """S_t[c, n] = exp(dt_t[c] A[c, n]) S_(t-1)[c, n] + dt_t[c] x_t[c] B_t[n];  y_t[c] = sum_n S_t[c, n] C_t[n] + Dskip[c] x_t[c].
    x, dt [T, E]; A [E, N]; B, C [T, N]."""
    T, E = x.shape
    S = torch.zeros(E, A.shape[1], dtype=F)
    y = torch.zeros(T, E, dtype=F)
    for t in range(T):
        S = torch.exp(dt[t].unsqueeze(1) * A) * S + (dt[t] * x[t]).unsqueeze(1) * B[t].unsqueeze(0)
        y[t] = S @ C[t] + Dskip * x[t]
    return y


def mamba_mixer(h, m, W, p):
    """in-projection [x | z]; x through a causal convolution and silu; step sizes, input and output maps from x; the
    scan; times silu(z); out-projection."""
    E, N, K = m["inner"], m["state"], m["dt_rank"]
    xz = h @ W[p + "in"].T
    x, z = xz[:, :E], xz[:, E:]
    x = silu(causal_conv(x, W[p + "conv"], W[p + "conv.b"]))
    low = x @ W[p + "x"].T
    dt = torch.nn.functional.softplus(low[:, :K] @ W[p + "dt"].T + W[p + "dt.b"])
    y = selective_scan(x, dt, -torch.exp(W[p + "A_log"]), low[:, K:K + N], low[:, K + N:K + 2 * N], W[p + "D"])
    return (y * silu(z)) @ W[p + "o"].T


# ---- feed-forwards ----------------------------------------------------------------------------------------------
def gated_unit(h, W, p, act):
    return (act(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def dense_ff(h, W, p):
    return gated_unit(h, W, p, torch.relu)


def routed_ff(h, mlp, W, p, margins=None):
    """Each token goes to the ``top`` experts of largest sigmoid(router) score; an expert sees score * h; their outputs
    add up, without renormalising, together with the shared expert's.  ``margins`` (a list) receives, per token, how far
    the last chosen expert's router output lies above the first one left out."""
    n, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
    z = h @ W[p + "router"].T
    scores = torch.sigmoid(z)
    if margins is not None:
        ranked = z.sort(dim=-1, descending=True).values
        margins.append(ranked[:, top - 1] - ranked[:, top] if top < n else torch.full((h.shape[0],), math.inf, dtype=F))
    out = torch.zeros(h.shape[0], W[p + "e0.down"].shape[0], dtype=F)
    for t in range(h.shape[0]):
        for e in torch.topk(scores[t], top).indices.tolist():
            out[t] += gated_unit((scores[t, e] * h[t]).unsqueeze(0), W, f"{p}e{e}.", silu)[0]
    if mlp.get("shared"):
        out = out + gated_unit(h, W, p + "shared.", silu)
    return out


# ---- the model --------------------------------------------------------------------------------------------------
def run_order(cfg):
    """(layer, pass number or None, first of its pass) for every layer run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None, False) for i in range(n)]
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    order = [(i, None, False) for i in range(a)]
    for t in range(times):
        order += [(i, t, i == a) for i in range(a, b)]
    return order + [(i, None, False) for i in range(b, n)]


def forward(tokens, cfg, W, return_layers=False, margins=None):
    """Logits [T, vocab] of one whole sequence; with ``return_layers`` also the stream after every layer run.  ``margins`` (a
    list) receives one tensor [T] per routed feed-forward that ran (see ``routed_ff``)."""
    W = {k: (v.to(F) if v.is_floating_point() else v) for k, v in W.items()}
    eps = float(cfg["norm"]["eps"])
    x0 = W["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    x = x0.clone()
    seen = []
    for i, t, first in run_order(cfg):
        layer = cfg["layers"][i]
        p = f"l{i}."
        if first:
            x = torch.cat([x, x0], -1) @ W["loop.in"].T + W["loop.step"][t]
        h = rms_norm(x, W[p + "norm1"], eps)
        if layer["type"] == "latent_attention":
            d = latent_attention(h, layer["mixer"], W, p + "mix.", eps)
        elif layer["type"] == "mamba1":
            d = mamba_mixer(h, layer["mixer"], W, p + "mix.")
        else:
            raise ValueError(layer["type"])
        x = x + rms_norm(d, W[p + "norm1b"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = rms_norm(x, W[p + "norm2"], eps)
            d = dense_ff(h, W, p + "mlp.") if mlp["kind"] == "dense" else routed_ff(h, mlp, W, p + "mlp.", margins)
            x = x + rms_norm(d, W[p + "norm2b"], eps)
        seen.append(x.clone())
    logits = rms_norm(x, W["final.norm"], eps) @ W["embed"].T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = float(cap) * torch.tanh(logits / float(cap))
    return (logits, torch.stack(seen)) if return_layers else logits
