"""The Demavik decoder, plainly: one function per mechanism, float64 throughout, a whole
sequence at a time, token by token where a mechanism is a recurrence, no cache, no batching.
It shares no code with the package; the engine's tests hold the kernels and the step function to it.

Notation: ``x`` [T, W] activations of one sequence (positions 0..T-1), ``w`` a dict of the
model's tensors by name (float64; integer tables excepted), ``cfg`` the dict of config.json,
``p`` a tensor-name prefix, ``m`` a layer's ``mixer`` entry.
"""

from __future__ import annotations

import math

import torch

F = torch.float64


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def silu(x):
    return x * torch.sigmoid(x)


def softplus(x):
    return torch.clamp(x, min=0.0) + torch.log1p(torch.exp(-x.abs()))


# ---------------------------------------------------------------------------------------------
# embedding
# ---------------------------------------------------------------------------------------------

def embed(cfg, w, tokens):
    """Token rows times a factor, plus a row of a second table chosen by a hash of (previous token, token); the first
    token of a sequence takes the table's last row."""
    e = cfg["embedding"]
    ids = torch.as_tensor(tokens, dtype=torch.long)
    x = w["embed"][ids] * float(e.get("scale", 1.0))
    b = e.get("bigram")
    if b:
        n, mp, mc = int(b["buckets"]), int(b["mul_prev"]), int(b["mul_cur"])
        rows = [n if t == 0 else (int(tokens[t - 1]) * mp + int(tokens[t]) * mc) % n for t in range(len(tokens))]
        x = x + w["bigram"][torch.tensor(rows, dtype=torch.long)]
    return x


# ---------------------------------------------------------------------------------------------
# rotation
# ---------------------------------------------------------------------------------------------

def rotary_frequencies(rot):
    """f_i = base^(-2i/dims); with ``scaling`` the long waves are slowed down: wavelengths beyond original/low by the
    whole factor, those below original/high not at all, those between by a blend that is linear in original/wavelength."""
    dims = int(rot["dims"])
    f = [float(rot["base"]) ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if sc:
        factor, low, high, orig = float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"])
        out = []
        for fi in f:
            wave = 2.0 * math.pi / fi
            if wave < orig / high:
                out.append(fi)
            elif wave > orig / low:
                out.append(fi / factor)
            else:
                s = (orig / wave - low) / (high - low)
                out.append((1.0 - s) * fi / factor + s * fi)
        f = out
    return torch.tensor(f, dtype=F)


def rotate(x, positions, rot):
    """x [T, heads, d]: element i of the first ``dims`` turns together with element i + dims/2 by position * f_i."""
    dims = int(rot["dims"])
    if not dims:
        return x
    half = dims // 2
    ang = positions.to(F)[:, None] * rotary_frequencies(rot)[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], dim=-1)


# ---------------------------------------------------------------------------------------------
# mixers
# ---------------------------------------------------------------------------------------------

def attention_keys_values(h, w, p, m, eps):
    """What an attention layer caches: keys after the norm over the whole projection and the rotation, and values."""
    T = h.shape[0]
    G, d = int(m.get("kv_heads") or m["heads"]), int(m["dim"])
    dv = int(m.get("vdim") or d)
    k = h @ w[p + "k"].T + w[p + "k.b"]
    v = h @ w[p + "v"].T + w[p + "v.b"]
    k = rms(k, eps) * w[p + "k.norm"]
    k = k.view(T, G, d)
    if m.get("rot"):
        k = rotate(k, torch.arange(T), m["rot"])
    return k, v.view(T, G, dv)


def softmax_attention(h, w, p, m, eps, kv):
    """Grouped-query causal attention with biased projections, an RMS norm over the whole query (and key) projection
    before the heads are split, rotation of part of each head; ``kv``: keys and values (of this or of another layer)."""
    T = h.shape[0]
    H, d = int(m["heads"]), int(m["dim"])
    dv = int(m.get("vdim") or d)
    k, v = kv
    G = k.shape[1]
    q = h @ w[p + "q"].T + w[p + "q.b"]
    q = (rms(q, eps) * w[p + "q.norm"]).view(T, H, d)
    if m.get("rot"):
        q = rotate(q, torch.arange(T), m["rot"])
    causal = torch.arange(T)[None, :] <= torch.arange(T)[:, None]
    out = torch.zeros(T, H, dv, dtype=F)
    for a in range(H):
        g = a // (H // G)
        s = (q[:, a] @ k[:, g].T) * float(m["scale"])
        s = s.masked_fill(~causal, -math.inf)
        out[:, a] = torch.softmax(s, dim=-1) @ v[:, g]
    return out.reshape(T, H * dv) @ w[p + "o"].T


def gated_linear_attention(h, w, p, m, eps):
    """Per head a matrix S [dim, vdim] that every token first shrinks row by row (a decay per key channel) and then adds
    k v^T to; the token reads S^T q.  The heads' outputs are RMS-normed one by one with a shared weight, gated and mapped out."""
    T = h.shape[0]
    H, d, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    q = (h @ w[p + "q"].T).view(T, H, d) * d ** -0.5
    k = (h @ w[p + "k"].T).view(T, H, d)
    v = (h @ w[p + "v"].T).view(T, H, dv)
    z = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "a2.b"]
    alpha = torch.sigmoid(z).pow(1.0 / float(m["tau"])).view(T, H, d)
    S = torch.zeros(H, d, dv, dtype=F)
    o = torch.zeros(T, H, dv, dtype=F)
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = rms(o, eps) * w[p + "norm"]
    return (o.reshape(T, H * dv) * silu(h @ w[p + "g"].T)) @ w[p + "o"].T


def causal_convolution(u, taps_w, bias):
    """Per channel over time: y_t = b + sum_j w[:, j] u_(t - taps + 1 + j), zeros before the first token."""
    T, C = u.shape
    taps = taps_w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=F), u], dim=0)
    y = bias.expand(T, C).clone()
    for j in range(taps):
        y = y + padded[j:j + T] * taps_w[:, j]
    return y


def selective_scan(h, w, p, m):
    """A state S [inner, state] per sequence: every channel c decays its row by exp(dt_c A[c, :]) and adds dt_c x_c B;
    the token reads S C + D x per channel, gated by silu(z)."""
    T = h.shape[0]
    inner, N, R = int(m["inner"]), int(m["state"]), int(m["dt_rank"])
    xz = h @ w[p + "in"].T
    x, z = xz[:, :inner], xz[:, inner:]
    x = silu(causal_convolution(x, w[p + "conv"], w[p + "conv.b"]))
    low = x @ w[p + "x"].T
    dt = softplus(low[:, :R] @ w[p + "dt"].T + w[p + "dt.b"])           # [T, inner]
    B, C = low[:, R:R + N], low[:, R + N:R + 2 * N]
    A = -torch.exp(w[p + "A_log"])                                       # [inner, N]
    S = torch.zeros(inner, N, dtype=F)
    y = torch.zeros(T, inner, dtype=F)
    for t in range(T):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * B[t][None, :]
        y[t] = S @ C[t] + w[p + "D"] * x[t]
    return (y * silu(z)) @ w[p + "o"].T


# ---------------------------------------------------------------------------------------------
# feed-forward
# ---------------------------------------------------------------------------------------------

def routed_experts(h, w, p, mlp):
    """Router logits with a bias; the ``top`` largest choose the experts; their weights are the softmax over the chosen
    logits alone; the weighted sum of the chosen experts' outputs."""
    E, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
    z = h @ w[p + "router"].T + w[p + "router.b"]
    best = torch.topk(z, top, dim=-1)
    weights = torch.softmax(best.values, dim=-1)
    y = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j, e in enumerate(best.indices[t].tolist()):
            pe = f"{p}e{e}."
            y[t] += weights[t, j] * ((silu(h[t] @ w[pe + "gate"].T) * (h[t] @ w[pe + "up"].T)) @ w[pe + "down"].T)
    return y


# ---------------------------------------------------------------------------------------------
# the model
# ---------------------------------------------------------------------------------------------

def forward(cfg, w, tokens, keep=None):
    """Logits [T, vocab] of one sequence; ``keep``: a list that receives the residual stream after every layer."""
    eps = float(cfg["norm"]["eps"])
    mult = float(cfg.get("residual_mult", 1.0))
    x = embed(cfg, w, tokens)
    cached = {}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        kind = layer["type"]
        if kind == "attention":
            src = m.get("kv_from")
            if src is None:
                cached[i] = attention_keys_values(x, w, p + "mix.", m, eps)
                src = i
            y = softmax_attention(x, w, p + "mix.", m, eps, cached[int(src)])
        elif kind == "gla":
            y = gated_linear_attention(x, w, p + "mix.", m, eps)
        elif kind == "mamba1":
            y = selective_scan(x, w, p + "mix.", m)
        else:
            raise ValueError(kind)
        # the norm stands on the sublayer's output only; the sublayer reads the stream as it is
        x = x + mult * rms(y, eps) * w[p + "norm1"]
        if layer.get("mlp") is not None:
            y = routed_experts(x, w, p + "mlp.", layer["mlp"])
            x = x + mult * rms(y, eps) * w[p + "norm2"]
        if keep is not None:
            keep.append(x.clone())
    return (rms(x, eps) * w["final.norm"]) @ w["head"].T
