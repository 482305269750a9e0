"""Plain, slow Murutar in float64 on the CPU: one function per mechanism, written from the
design's equations and sharing no code with the package.  ``forward`` runs whole sequences
token by token where a mechanism is sequential and returns the logits of every position and
the residual stream after every layer.

Notation: h is what a sublayer reads, p a position, W x a stored [out, in] matrix applied to x.
"""
from __future__ import annotations

import math

import torch

F = torch.float64


def layer_norm(x, w, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w


def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def rotate_halves(x, positions, dims, base):
    """x [T, heads, dim]: dimension i < dims/2 of every head is paired with i + dims/2 and the pair
    turned by the angle p * base^(-2i/dims); dimensions from ``dims`` on pass unchanged."""
    if not dims:
        return x
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F)
    a = positions.to(F)[:, None] * f[None, :]  # [T, half]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def sink_window_attention(q, k, v, scale, window):
    """q [T, H, d], k [T, G, d], v [T, G, dv] of one sequence from position 0.  Query i sees keys j
    with 0 <= i - j < window (window 0: every j <= i); weights exp(s_j) / (1 + sum exp(s_j))."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=F)
    for i in range(T):
        lo = max(0, i - window + 1) if window else 0
        for h in range(H):
            g = h // (H // G)
            s = (k[lo:i + 1, g] @ q[i, h]) * scale
            m = max(float(s.max()), 0.0)
            e = torch.exp(s - m)
            p = e / (math.exp(-m) + e.sum())
            out[i, h] = p @ v[lo:i + 1, g]
    return out


def lightning_recurrence(q, k, v, decay, state=None):
    """q, k [T, H, d], v [T, H, dv]: S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t."""
    T, H, d = q.shape
    S = torch.zeros(H, d, v.shape[2], dtype=F) if state is None else state.clone()
    lam = torch.tensor(decay, dtype=F)[:, None, None]
    out = torch.zeros(T, H, v.shape[2], dtype=F)
    for t in range(T):
        S = lam * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return out, S


def lightning_mixer(h, w, p, m, eps):
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[p + "q"].T).view(T, H, d)
    k = silu(h @ w[p + "k"].T).view(T, H, d)
    v = silu(h @ w[p + "v"].T).view(T, H, dv)
    o, _ = lightning_recurrence(q, k, v, m["decay"])
    o = rms_norm(o.reshape(T, H * dv), w[p + "norm"], eps) * torch.sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def attention_mixer(h, w, p, m, positions, shared):
    """``shared``: carries the first value-mixing layer's values to the later ones."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).view(T, H, d)
    k = (h @ w[p + "k"].T).view(T, G, d)
    v = (h @ w[p + "v"].T).view(T, G, dv)
    rot = m.get("rot") or {}
    q = rotate_halves(q, positions, rot.get("dims", 0), rot.get("base", 1.0))
    k = rotate_halves(k, positions, rot.get("dims", 0), rot.get("base", 1.0))
    if m.get("v_mix"):
        if "v_first" not in shared:
            shared["v_first"] = v
        else:
            lam = w[p + "vmix"]
            v = (1.0 - lam) * v + lam * shared["v_first"]
    window = (m.get("mask") or {}).get("size", 0) or 0
    o = sink_window_attention(q, k, v, m["scale"], window)
    return o.reshape(T, H * dv) @ w[p + "o"].T


def dense_ff(h, w, p, mlp):
    lim = mlp["limit"]
    g = torch.clamp(h @ w[p + "gate"].T, max=lim)
    u = torch.clamp(h @ w[p + "up"].T, -lim, lim)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


ROUTING_MARGINS = None  # a list: route() appends (token, how far the choice was from going the other way)
_TOKEN = 0  # the token moe_ff is at


def route(scores, router):
    """scores [experts] -> indices of the chosen experts: the ``top`` largest scores among the
    experts of the ``keep`` groups (equal runs of neighbours) whose largest score is largest."""
    E, n_groups, keep, top = router["experts"], router["groups"]["count"], router["groups"]["keep"], router["top"]
    per = E // n_groups
    best = scores.view(n_groups, per).max(dim=1).values
    kept = torch.topk(best, keep).indices
    allowed = torch.zeros(E, dtype=torch.bool)
    for g in kept.tolist():
        allowed[g * per:(g + 1) * per] = True
    masked = torch.where(allowed, scores, torch.full_like(scores, -1.0))
    chosen = torch.topk(masked, top).indices
    if ROUTING_MARGINS is not None:
        # log-ratio (= difference of router logits) between the last one in and the first one out
        if keep < n_groups:
            order = torch.sort(best, descending=True).values
            ROUTING_MARGINS.append((_TOKEN, float(torch.log(order[keep - 1] / order[keep]))))
        order = torch.sort(masked, descending=True).values
        if top < int(allowed.sum()):
            ROUTING_MARGINS.append((_TOKEN, float(torch.log(order[top - 1] / order[top]))))
    return chosen


def moe_ff(h, w, p, mlp):
    router = mlp["router"]
    out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=F)
    global _TOKEN
    for t in range(h.shape[0]):
        _TOKEN = t
        s = torch.softmax(w[p + "router"] @ h[t], dim=0)
        for e in route(s, router).tolist():
            a = torch.relu(w[f"{p}e{e}.up"] @ h[t]) ** 2
            out[t] += s[e] * (w[f"{p}e{e}.down"] @ a)
    return out


def side_input(x, tokens, w, layer, dim, eps):
    e = w["side.embed"][tokens][:, layer * dim:(layer + 1) * dim]
    g = gelu_tanh(x @ w[f"l{layer}.side.gate"].T) * e
    y = g @ w[f"l{layer}.side.proj"].T
    return rms_norm(y, w[f"l{layer}.side.norm"], eps)


def forward(cfg: dict, weights: dict, tokens: list):
    """Returns (logits [T, vocab], residual stream after every layer [L, T, width]) in float64."""
    w = {n: t.to(F) for n, t in weights.items()}
    eps = cfg["norm"]["eps"]
    tok = torch.tensor(tokens, dtype=torch.long)
    positions = torch.arange(len(tokens))
    x = w["embed"][tok] * cfg["embedding"]["scale"]
    side = cfg.get("token_side")
    shared: dict = {}
    streams = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = layer_norm(x, w[p + "norm1"], eps)
        if layer["type"] == "attention":
            y = attention_mixer(h, w, p + "mix.", layer["mixer"], positions, shared)
        elif layer["type"] == "lightning":
            y = lightning_mixer(h, w, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        x = x + y * w[p + "ls1"] * torch.sigmoid(h @ w[p + "rg1"].T + w[p + "rg1.b"])
        mlp = layer.get("mlp")
        if mlp is not None:
            h = layer_norm(x, w[p + "norm2"], eps)
            y = dense_ff(h, w, p + "mlp.", mlp) if mlp["kind"] == "dense" else moe_ff(h, w, p + "mlp.", mlp)
            x = x + y * w[p + "ls2"] * torch.sigmoid(h @ w[p + "rg2"].T + w[p + "rg2.b"])
        if side:
            x = x + side_input(x, tok, w, i, side["dim"], eps)
        streams.append(x)
    h = layer_norm(x, w["final.norm"], eps)
    logits = h @ w["embed"].T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return logits, torch.stack(streams)
