"""Plain, slow implementation of the Puludra decoder on the CPU: the oracle of the tests.

One function per mechanism, written from the equations, token by token where the mechanism is a
recurrence.  It shares no code with the package: weights come as a dict of tensors by checkpoint
name, the configuration as the dict of config.json.  Everything runs in one floating-point type
(float64 unless asked otherwise).

Layer (norm after the sum):   x <- N1(alpha x + mixer(x));   x <- N2(alpha x + ff(x))
RMS norm:                     N(x) = x / sqrt(mean(x^2) + eps) * w
"""
from __future__ import annotations

import math

import torch


def rms_norm(x, w, eps):
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if w is None else y * w


def angles(positions, base, dims, dtype):
    """[T, dims/2]: position * base^(-2i/dims)."""
    i = torch.arange(dims // 2, dtype=dtype)
    freq = base ** (-2.0 * i / dims)
    return positions.to(dtype)[:, None] * freq[None, :]


def rotate_interleaved(x, positions, base, dims):
    """x [T, heads, d]: dimension 2i is turned together with 2i+1, over the first ``dims``."""
    a = angles(positions, base, dims, x.dtype)
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    out = x.clone()
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def rotate_halves(x, positions, base, dims):
    """x [T, heads, d]: dimension i is turned together with i + dims/2, over the first ``dims``."""
    a = angles(positions, base, dims, x.dtype)
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    out = x.clone()
    half = dims // 2
    u, v = x[..., :half], x[..., half:dims]
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


def latent_attention(h, w, m, eps, positions):
    """h [T, width]; ``w``: this mixer's tensors by their short names; ``m``: its sizes."""
    T = h.shape[0]
    H, d, r, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    cq = rms_norm(h @ w["dq"].T, w["dq.norm"], eps)
    q = (cq @ w["uq"].T).view(T, H, d + r)
    q_plain, q_rot = q[..., :d], q[..., d:]
    down = h @ w["dkv"].T
    c = rms_norm(down[:, :R], w["dkv.norm"], eps)
    k_rot = down[:, None, R:]  # one head, shared
    rot = m["rot"]
    q_rot = rotate_interleaved(q_rot, positions, rot["base"], rot["dims"])
    k_rot = rotate_interleaved(k_rot, positions, rot["base"], rot["dims"])
    k_plain = (c @ w["uk"].T).view(T, H, d)
    v = (c @ w["uv"].T).view(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        for a in range(H):
            s = (k_plain[: t + 1, a] @ q_plain[t, a] + k_rot[: t + 1, 0] @ q_rot[t, a]) * m["scale"]
            p = torch.softmax(s, dim=0)
            out[t, a] = p @ v[: t + 1, a]
    return out.reshape(T, H * dv) @ w["o"].T


def hgrn2(h, w, m, eps, positions=None):
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = torch.nn.functional.silu(h @ w["q"].T).view(T, H, d)
    v = (h @ w["v"].T).view(T, H, dv)
    low = w["lower"]
    f = (low + (1.0 - low) * torch.sigmoid(h @ w["f"].T + w["f.b"])).view(T, H, d)
    S = torch.zeros(H, d, dv, dtype=h.dtype)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        S = f[t][:, :, None] * S + (1.0 - f[t])[:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", S, q[t])
    out = rms_norm(out, w["norm"], eps)
    return out.reshape(T, H * dv) @ w["o"].T


def retention(h, w, m, eps, positions):
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    rot = m["rot"]
    q = rotate_halves((h @ w["q"].T).view(T, H, d), positions, rot["base"], rot["dims"])
    k = rotate_halves((h @ w["k"].T).view(T, H, d), positions, rot["base"], rot["dims"]) * d ** -0.5
    v = (h @ w["v"].T).view(T, H, dv)
    decay = torch.tensor(m["decay"], dtype=h.dtype)
    S = torch.zeros(H, d, dv, dtype=h.dtype)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", S, q[t])
    out = rms_norm(out, None, eps).reshape(T, H * dv)
    return (out * torch.nn.functional.silu(h @ w["g"].T)) @ w["o"].T


def xielu(z, p, q):
    sp = torch.nn.functional.softplus
    pos = sp(p) * z * z + z / 2
    neg = (0.5 + sp(q)) * (torch.expm1(z) - z) + z / 2
    return torch.where(z > 0, pos, neg)


def dense_ff(h, w):
    return xielu(h @ w["up"].T, w["act"][0], w["act"][1]) @ w["down"].T


MIXERS = {"latent_attention": latent_attention, "hgrn2": hgrn2, "retention": retention}


def layer_tensors(weights, index, part, dtype):
    prefix = f"l{index}.{part}."
    return {k[len(prefix):]: v.to(dtype) for k, v in weights.items() if k.startswith(prefix)}


def forward(weights, config, ids, dtype=torch.float64, keep_layers=False):
    """Logits [T, vocab] of one sequence from position 0 (and the stream after every layer run)."""
    ids = torch.as_tensor(ids, dtype=torch.long)
    positions = torch.arange(ids.shape[0])
    eps, alpha = config["norm"]["eps"], config["postln_alpha"]
    x = weights["embed"].to(dtype)[ids]
    kept = []
    for i, entry in enumerate(config["layers"]):
        src = i
        while "weights_of" in config["layers"][src]:
            src = config["layers"][src]["weights_of"]
        mix = layer_tensors(weights, src, "mix", dtype)
        y = MIXERS[entry["type"]](x, mix, entry["mixer"], eps, positions)
        x = rms_norm(alpha * x + y, weights[f"l{src}.norm1"].to(dtype), eps)
        if entry.get("mlp") is not None:
            y = dense_ff(x, layer_tensors(weights, src, "mlp", dtype))
            x = rms_norm(alpha * x + y, weights[f"l{src}.norm2"].to(dtype), eps)
        kept.append(x)
    logits = rms_norm(x, weights["final.norm"].to(dtype), eps) @ weights["head"].to(dtype).T
    return (logits, torch.stack(kept)) if keep_layers else logits


def greedy_generate(weights, config, prompt, n, dtype=torch.float64):
    """n greedy tokens and, for each, the gap between the two largest logits."""
    ids, out, gaps = list(prompt), [], []
    for _ in range(n):
        logits = forward(weights, config, ids, dtype)[-1]
        top = torch.topk(logits, 2).values
        out.append(int(logits.argmax()))
        gaps.append(float(top[0] - top[1]))
        ids.append(out[-1])
    return out, gaps


def tensor_shapes(config):
    """name -> shape of every tensor a model of this configuration has."""
    W, V = config["width"], config["vocab"]
    shapes = {"embed": (V, W), "final.norm": (W,), "head": (V, W)}
    for i, e in enumerate(config["layers"]):
        if "weights_of" in e:
            continue
        m, p = e["mixer"], f"l{i}."
        shapes[p + "norm1"] = (W,)
        H, d, dv = m["heads"], m["dim"], m["vdim"]
        if e["type"] == "retention":
            for n in "qkg":
                shapes[p + "mix." + n] = (H * (dv if n == "g" else d), W)
            shapes[p + "mix.v"] = (H * dv, W)
            shapes[p + "mix.o"] = (W, H * dv)
        elif e["type"] == "hgrn2":
            shapes[p + "mix.q"] = shapes[p + "mix.f"] = (H * d, W)
            shapes[p + "mix.f.b"] = shapes[p + "mix.lower"] = (H * d,)
            shapes[p + "mix.v"] = (H * dv, W)
            shapes[p + "mix.norm"] = (dv,)
            shapes[p + "mix.o"] = (W, H * dv)
        elif e["type"] == "latent_attention":
            r, R, Q = m["rot_dim"], m["kv_rank"], m["q_rank"]
            shapes[p + "mix.dq"] = (Q, W)
            shapes[p + "mix.dq.norm"] = (Q,)
            shapes[p + "mix.uq"] = (H * (d + r), Q)
            shapes[p + "mix.dkv"] = (R + r, W)
            shapes[p + "mix.dkv.norm"] = (R,)
            shapes[p + "mix.uk"] = (H * d, R)
            shapes[p + "mix.uv"] = (H * dv, R)
            shapes[p + "mix.o"] = (W, H * dv)
        if e.get("mlp") is not None:
            shapes[p + "norm2"] = (W,)
            shapes[p + "mlp.up"] = (e["mlp"]["ff"], W)
            shapes[p + "mlp.down"] = (W, e["mlp"]["ff"])
            shapes[p + "mlp.act"] = (2,)
    return shapes


def random_weights(config, seed, std=None):
    """Random tensors, rounded to bfloat16 values (kept as float32)."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(config).items():
        fan_in = shape[-1]
        if name.endswith(("norm1", "norm2", ".norm")) :
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        elif name.endswith("lower"):
            t = torch.rand(shape, generator=g) * 0.9
        elif name.endswith("act"):
            t = torch.randn(shape, generator=g) * 0.5
        elif name.endswith("f.b"):
            t = torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) * (std if std is not None else 1.0 / math.sqrt(fan_in))
        out[name] = t.to(torch.bfloat16).to(torch.float32)
    return out
