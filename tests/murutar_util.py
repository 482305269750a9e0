"""Tiny Murutar configurations, weights and model folders for the tests.  The list of tensors is
derived here from the configuration (not from the package's builder), the weights are drawn with
torch's generator and written with the package's safetensors writer."""
import copy
import json
import os

import torch


def attention(heads, kv_heads, dim, vdim, window=None, rot=None, base=10000.0, v_mix=False, scale=None, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
         "scale": scale if scale is not None else dim ** -0.5, "v_mix": v_mix}
    if window is not None:
        m["mask"] = {"size": window}
    if rot:
        m["rot"] = {"base": base, "dims": rot}
    return {"type": "attention", "mixer": m, "mlp": mlp}


def lightning(heads, dim, vdim, decay, mlp=None):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}, "mlp": mlp}


def dense(ff, limit=1.0):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(experts, top, ff, groups=1, keep=1):
    return {"kind": "moe", "expert": {"ff": ff},
            "router": {"experts": experts, "top": top, "groups": {"count": groups, "keep": keep}}}


def model(width, vocab, layers, eps=1e-6, scale=None, softcap=None, side=None):
    d = {"architecture": "Murutar", "vocab": vocab, "width": width, "embedding": {"scale": scale or width ** 0.5},
         "norm": {"eps": eps}, "layers": layers}
    if softcap:
        d["logit_softcap"] = softcap
    if side:
        d["token_side"] = {"dim": side}
    return d


CONFIGS = {
    # both mixers and both feed-forwards, a layer without a feed-forward, a window shorter than a
    # page, one that is no multiple of it, a layer without window, rotation or blending; the first
    # blending layer is not the first attention layer
    "mix": dict(config=model(64, 160, [
        lightning(3, 8, 12, [0.9, 0.99, 1.0], mlp=moe(6, 2, 24, groups=3, keep=2)),
        attention(2, 2, 8, 8, mlp=dense(40, limit=0.7)),
        attention(4, 2, 16, 8, window=20, rot=8, v_mix=True, mlp=dense(40, limit=2.5)),
        attention(6, 2, 16, 8, window=7, rot=16, base=50.0, v_mix=True),
        lightning(1, 16, 8, [0.95], mlp=dense(48)),
        attention(2, 2, 24, 8, window=40, rot=12, v_mix=True, mlp=moe(4, 1, 16)),
    ], softcap=20.0, side=5), seed=21, page_size=16),
    # nothing a multiple of 8, one query head per key head, no softcap, no token input, every
    # group kept, more experts chosen than a group holds
    "odd": dict(config=model(52, 211, [
        attention(5, 5, 6, 10, window=33, rot=4, base=300.0, v_mix=True, scale=0.5, mlp=moe(9, 4, 14, groups=3, keep=3)),
        lightning(1, 10, 7, [1.0], mlp=dense(30, limit=1.5)),
        attention(5, 5, 10, 10, window=9, rot=10, v_mix=True, mlp=None),
    ], eps=3e-6, scale=3.0), seed=22, page_size=8),
    # sizes the tensor-core products take; nine query heads per key head, values wider than keys,
    # a window of exactly two pages, state rows split over several threads
    "wide": dict(config=model(256, 384, [
        attention(18, 2, 64, 128, window=64, rot=32, base=1e6, v_mix=True, mlp=dense(512)),
        lightning(2, 160, 40, [0.999, 0.8], mlp=moe(16, 3, 128, groups=4, keep=2)),
        attention(8, 2, 32, 128, window=100, rot=16, v_mix=True, mlp=moe(8, 2, 64, groups=2, keep=1)),
        lightning(4, 32, 64, [0.9, 0.99, 0.999, 1.0], mlp=dense(384, limit=1.0)),
    ], softcap=30.0, side=16), seed=23, page_size=32),
    "only_attention": dict(config=model(48, 96, [attention(4, 2, 8, 12, window=24, rot=8, mlp=dense(64))], side=4),
                           seed=24, page_size=16),
    "only_lightning": dict(config=model(48, 96, [lightning(3, 8, 12, [0.9, 0.99, 0.97], mlp=moe(4, 2, 32, groups=2, keep=2))],
                                        softcap=15.0), seed=25, page_size=16),
}


def tensor_shapes(config):
    """name -> shape of every tensor a checkpoint of this configuration holds."""
    W, V = config["width"], config["vocab"]
    L = len(config["layers"])
    side = (config.get("token_side") or {}).get("dim", 0)
    shapes = {"embed": (V, W), "final.norm": (W,)}
    if side:
        shapes["side.embed"] = (V, L * side)
    for i, e in enumerate(config["layers"]):
        p, m = f"l{i}.", e["mixer"]
        shapes.update({p + "norm1": (W,), p + "ls1": (W,), p + "rg1": (W, W), p + "rg1.b": (W,)})
        if e["type"] == "attention":
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            shapes.update({p + "mix.q": (H * d, W), p + "mix.k": (G * d, W), p + "mix.v": (G * dv, W),
                           p + "mix.o": (W, H * dv)})
            if m.get("v_mix"):
                shapes[p + "mix.vmix"] = ()
        else:
            H, d, dv = m["heads"], m["dim"], m["vdim"]
            shapes.update({p + "mix.q": (H * d, W), p + "mix.k": (H * d, W), p + "mix.v": (H * dv, W),
                           p + "mix.g": (H * dv, W), p + "mix.o": (W, H * dv), p + "mix.norm": (H * dv,)})
        mlp = e.get("mlp")
        if mlp is not None:
            shapes.update({p + "norm2": (W,), p + "ls2": (W,), p + "rg2": (W, W), p + "rg2.b": (W,)})
            if mlp["kind"] == "dense":
                shapes.update({p + "mlp.gate": (mlp["ff"], W), p + "mlp.up": (mlp["ff"], W), p + "mlp.down": (W, mlp["ff"])})
            else:
                shapes[p + "mlp.router"] = (mlp["router"]["experts"], W)
                for x in range(mlp["router"]["experts"]):
                    shapes[f"{p}mlp.e{x}.up"] = (mlp["expert"]["ff"], W)
                    shapes[f"{p}mlp.e{x}.down"] = (W, mlp["expert"]["ff"])
        if side:
            shapes.update({p + "side.gate": (side, W), p + "side.proj": (W, side), p + "side.norm": (W,)})
    return shapes


def random_weights(config, seed):
    """Weights as float32 tensors holding bfloat16 values."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(config).items():
        last = name.split(".")[-1]
        if last in ("norm1", "norm2") or name in ("final.norm",) or name.endswith(("mix.norm", "side.norm")):
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        elif last in ("ls1", "ls2"):
            t = 0.3 + 0.5 * torch.rand(shape, generator=g)
        elif last == "b":
            t = 0.5 * torch.randn(shape, generator=g)
        elif last == "vmix":
            t = 0.25 + 0.5 * torch.rand(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g) / shape[1] ** 0.5
        elif name == "side.embed":
            t = torch.randn(shape, generator=g)
        elif last == "router":
            t = 2.0 * torch.randn(shape, generator=g) / shape[1] ** 0.5
        else:
            t = torch.randn(shape, generator=g) / shape[-1] ** 0.5
        out[name] = t.to(torch.bfloat16).float()
    return out


def sharpen(config, weights):
    """Makes far tokens and window edges matter: attention queries are scaled up so that every
    softmax falls on one or two keys of the window (and beats the sink), and the keys of the linear
    attention grow so that what the state has held for long still shows."""
    out = dict(weights)
    for i, e in enumerate(config["layers"]):
        if e["type"] == "attention":
            out[f"l{i}.mix.q"] = (weights[f"l{i}.mix.q"] * 12.0).to(torch.bfloat16).float()
        else:
            out[f"l{i}.mix.k"] = (weights[f"l{i}.mix.k"] * 3.0).to(torch.bfloat16).float()
    return out


def make_folder(folder, name, sharp=False):
    """Writes config.json and model.safetensors (bfloat16); returns (config, weights as float32)."""
    from dispec_b200.weights import write_safetensors

    spec = CONFIGS[name]
    config = copy.deepcopy(spec["config"])
    weights = random_weights(config, spec["seed"])
    if sharp:
        weights = sharpen(config, weights)
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(config, f)
    write_safetensors(os.path.join(folder, "model.safetensors"),
                      {k: v.to(torch.bfloat16) for k, v in weights.items()})
    return config, weights
