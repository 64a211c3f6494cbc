"""The Pifazen decoder, plainly: one function per mechanism, float64 throughout, a whole
sequence at a time, token by token where a mechanism is a recurrence, no cache, no batching.
It shares no code with the package; the engine's tests hold the kernels and the step function to it.

Notation: ``x`` [T, W] activations of one sequence (positions 0..T-1), ``w`` a dict of the
model's tensors by name (float64), ``cfg`` the dict of config.json, ``p`` a tensor-name prefix,
``m`` a layer's ``mixer`` entry.
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


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def offset_norm(x, weight, eps):
    """The layer's norm: the weight is stored around zero."""
    return rms(x, eps) * (1.0 + weight)


# ---------------------------------------------------------------------------------------------
# rotation
# ---------------------------------------------------------------------------------------------

def rotary_frequencies(rot):
    """(f_i, magnitude): f_i = base^(-2i/dims); with ``scaling`` the waves that do not fit ``original`` positions ``slow``
    times are divided by ``factor``, those that fit more than ``fast`` times stay, the ones between are blended by the
    index of the pair; cosines and sines then carry the magnitude 0.1 ln(factor) + 1."""
    dims = int(rot["dims"])
    base = float(rot["base"])
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if not sc:
        return torch.tensor(f, dtype=F), 1.0
    factor, orig, fast, slow = float(sc["factor"]), float(sc["original"]), float(sc["fast"]), float(sc["slow"])

    def index_of(turns):
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(index_of(fast)), 0)
    hi = min(math.ceil(index_of(slow)), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * ramp + fi * (1.0 - ramp))
    return torch.tensor(out, dtype=F), 0.1 * math.log(factor) + 1.0


def rotate_pairs(x, positions, rot):
    """x [T, heads, d]: elements 2i and 2i + 1 of the first ``dims`` turn together by position * f_i."""
    dims = int(rot["dims"])
    f, mag = rotary_frequencies(rot)
    ang = positions.to(F)[:, None] * f[None, :]
    c, s = (torch.cos(ang) * mag)[:, None, :], (torch.sin(ang) * mag)[:, None, :]
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


# ---------------------------------------------------------------------------------------------
# mixers
# ---------------------------------------------------------------------------------------------

def causal_conv(u, weight):
    """u [T, C], weight [C, taps]: out_t = sum_j weight[:, j] u_(t - taps + 1 + j), zeros before the start."""
    T, C = u.shape
    taps = weight.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=F), u], dim=0)
    out = torch.zeros(T, C, dtype=F)
    for j in range(taps):
        out = out + padded[j:j + T] * weight[:, j][None, :]
    return out


def channel_delta(h, w, p, m, eps):
    """The gated delta rule with a decay per head and key channel."""
    T = h.shape[0]
    H, d = int(m["heads"]), int(m["dim"])
    G = int(m.get("kv_heads") or H)
    dv = int(m.get("vdim") or d)
    q = silu(causal_conv(h @ w[p + "q"].T, w[p + "q.conv"])).view(T, G, d)
    k = silu(causal_conv(h @ w[p + "k"].T, w[p + "k.conv"])).view(T, G, d)
    v = silu(causal_conv(h @ w[p + "v"].T, w[p + "v.conv"])).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[p + "b"].T)                                        # [T, H]
    dt = softplus((h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "dt_bias"]).view(T, H, d)
    g = torch.exp(-torch.exp(w[p + "A_log"])[None, :, None] * dt)                 # [T, H, d]
    o = torch.zeros(T, H, dv, dtype=F)
    for a in range(H):
        kv = a // (H // G)
        S = torch.zeros(d, dv, dtype=F)
        for t in range(T):
            S = g[t, a][:, None] * S
            u = beta[t, a] * (v[t, a] - S.T @ k[t, kv])
            S = S + torch.outer(k[t, kv], u)
            o[t, a] = S.T @ q[t, kv]
    gate = torch.sigmoid((h @ w[p + "g1"].T) @ w[p + "g2"].T).view(T, H, dv)
    o = rms(o, eps) * w[p + "norm"] * gate
    return o.reshape(T, H * dv) @ w[p + "o"].T


def latent_attention(h, w, p, m, eps, kind):
    """Attention whose keys and values come from one latent per token, with one rotated key part shared by the heads.
    ``kind`` "latent_attention": queries through a latent of their own, a gate per output element;
    "latent_attention_2": queries straight from the input, a gate per head."""
    T = h.shape[0]
    H, d, dr, dv, R = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    pos = torch.arange(T)
    if kind == "latent_attention":
        cq = rms(h @ w[p + "dq"].T, eps) * w[p + "dq.norm"]
        q = cq @ w[p + "uq"].T
    else:
        q = h @ w[p + "q"].T
    q = q.view(T, H, d + dr)
    q_plain, q_rot = q[..., :d], rotate_pairs(q[..., d:], pos, m["rot"])
    low = h @ w[p + "dkv"].T
    c = rms(low[:, :R], eps) * w[p + "dkv.norm"]
    k_rot = rotate_pairs(low[:, None, R:], pos, m["rot"])[:, 0]                    # [T, dr]
    k_plain = (c @ w[p + "uk"].T).view(T, H, d)
    v = (c @ w[p + "uv"].T).view(T, H, dv)
    causal = pos[None, :] <= pos[:, None]
    out = torch.zeros(T, H, dv, dtype=F)
    for a in range(H):
        s = (q_plain[:, a] @ k_plain[:, a].T + q_rot[:, a] @ k_rot.T) * float(m["scale"])
        s = s.masked_fill(~causal, float("-inf"))
        out[:, a] = torch.softmax(s, dim=-1) @ v[:, a]
    gate = torch.sigmoid(h @ w[p + "g"].T)
    if kind == "latent_attention":
        out = out * gate.view(T, H, dv)
    else:
        out = out * gate[:, :, None]
    return out.reshape(T, H * dv) @ w[p + "o"].T


# ---------------------------------------------------------------------------------------------
# feed-forward
# ---------------------------------------------------------------------------------------------

def polynorm_feed_forward(h, w, p, eps):
    z = h @ w[p + "up"].T + w[p + "up.b"]
    a, b, c, e = (float(x) for x in w[p + "act"])
    y = a * rms(z, eps) + b * rms(z ** 2, eps) + c * rms(z ** 3, eps) + e
    return y @ w[p + "down"].T + w[p + "down.b"]


def route(h, w, p, mlp):
    """(ids [T, top], weights [T, top]) over experts and identity experts together."""
    r = mlp["router"]
    E, I, top = int(r["experts"]), int(r.get("identity") or 0), int(r["top"])
    n = E + I
    s = torch.softmax(h @ w[p + "router"].T, dim=-1)                               # [T, n]
    choice = s + w[p + "correction"]
    groups = r.get("groups")
    if groups:
        count, keep = int(groups["count"]), int(groups["keep"])
        best = choice.view(-1, count, n // count).max(dim=-1).values                # [T, count]
        kept = torch.zeros_like(best, dtype=torch.bool)
        # the best groups, the lower index first among equals
        order = torch.sort(best, dim=-1, descending=True, stable=True).indices[:, :keep]
        kept.scatter_(1, order, True)
        allowed = kept[:, :, None].expand(-1, -1, n // count).reshape(-1, n)
        choice = choice.masked_fill(~allowed, float("-inf"))
    ids = torch.sort(choice, dim=-1, descending=True, stable=True).indices[:, :top]
    chosen = torch.gather(s, 1, ids)
    weights = chosen / (chosen.sum(dim=-1, keepdim=True) + 1e-20) * float(r["scale"])
    return ids, weights


def expert(h, w, p, limit):
    g = torch.clamp(h @ w[p + "gate"].T, max=limit)
    u = torch.clamp(h @ w[p + "up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def mixture(h, w, p, mlp):
    E = int(mlp["router"]["experts"])
    limit = float(mlp["expert"]["limit"])
    ids, weights = route(h, w, p, mlp)
    y = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, wt in zip(ids[t].tolist(), weights[t]):
            y[t] += wt * (h[t] if e >= E else expert(h[t:t + 1], w, f"{p}e{e}.", limit)[0])
    return y


# ---------------------------------------------------------------------------------------------
# the model
# ---------------------------------------------------------------------------------------------

def layer(x, w, cfg, i):
    """x += ls1 * mixer(norm1(x)); x += ls2 * ff(norm2(x)); a layer with ``weights_of`` runs on that layer's tensors."""
    entry = cfg["layers"][i]
    src = entry.get("weights_of")
    p = f"l{i if src is None else src}."
    eps = float(cfg["norm"]["eps"])
    kind, m = entry["type"], entry["mixer"]
    h = offset_norm(x, w[p + "norm1"], eps)
    if kind == "channel_delta":
        y = channel_delta(h, w, p + "mix.", m, eps)
    elif kind in ("latent_attention", "latent_attention_2"):
        y = latent_attention(h, w, p + "mix.", m, eps, kind)
    else:
        raise ValueError(kind)
    x = x + w[p + "ls1"] * y
    mlp = entry.get("mlp")
    if mlp is not None:
        h = offset_norm(x, w[p + "norm2"], eps)
        y = polynorm_feed_forward(h, w, p + "mlp.", eps) if mlp["kind"] == "dense" else mixture(h, w, p + "mlp.", mlp)
        x = x + w[p + "ls2"] * y
    return x


def forward(cfg, w, tokens, streams=None):
    """Logits [T, vocab] of one sequence; ``streams`` (a list) takes the residual stream after every layer."""
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    for i in range(len(cfg["layers"])):
        x = layer(x, w, cfg, i)
        if streams is not None:
            streams.append(x.clone())
    return offset_norm(x, w["final.norm"], float(cfg["norm"]["eps"])) @ w["embed"].T
