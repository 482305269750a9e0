"""Tiny Puludra configurations and model folders for the tests.  Weights are drawn by the plain
implementation's own generator and written with the package's safetensors writer."""
import copy
import json
import os

import torch

import plain_puludra as plain


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, base=10000.0, scale=None, mlp=None):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
                      "q_rank": q_rank, "scale": scale if scale is not None else (dim + rot_dim) ** -0.5,
                      "rot": {"base": base, "dims": rot_dim}},
            "mlp": {"kind": "dense", "ff": mlp} if mlp else None}


def hgrn2(heads, dim, vdim, mlp=None):
    return {"type": "hgrn2", "mixer": {"heads": heads, "dim": dim, "vdim": vdim},
            "mlp": {"kind": "dense", "ff": mlp} if mlp else None}


def retention(heads, dim, vdim, decay, rot_dims, base=10000.0, mlp=None):
    return {"type": "retention",
            "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay),
                      "rot": {"base": base, "dims": rot_dims}},
            "mlp": {"kind": "dense", "ff": mlp} if mlp else None}


def again(layer, index):
    e = copy.deepcopy(layer)
    e["weights_of"] = index
    return e


def model(width, vocab, alpha, eps, layers):
    return {"architecture": "Puludra", "vocab": vocab, "width": width, "postln_alpha": alpha,
            "norm": {"eps": eps}, "layers": layers}


_LA = latent(2, 16, 8, 24, 40, 48, mlp=96)
_LB = latent(3, 12, 6, 10, 20, 28, base=300.0)
CONFIGS = {
    # every mixer, a layer that runs another's weights, feed-forwards on some layers only
    "mix": dict(config=model(64, 160, 1.5, 1e-5, [
        _LA, hgrn2(2, 16, 16), retention(3, 16, 32, [0.9, 0.99, 1.0], 8, mlp=72), again(_LA, 0)]),
        seed=11, page_size=16),
    # sizes no fast path takes (nothing a multiple of 8, one head, dim != vdim), alpha 1, a layer
    # that runs the weights of a LATER layer, the recurrent layers first
    "odd": dict(config=model(52, 211, 1.0, 3e-6, [
        hgrn2(5, 6, 9, mlp=30), again(_LB, 3), retention(1, 10, 7, [0.97], 6, base=50.0), _LB]),
        seed=12, page_size=8),
    # sizes the tensor-core products take; more heads than one block of the attention kernel holds,
    # a latent wider than one pass of its threads, state rows split over eight threads
    "wide": dict(config=model(256, 384, 2.5, 1e-6, [
        retention(2, 64, 48, [0.995, 0.9], 64, base=1e6), latent(10, 32, 16, 32, 192, 96, base=5e5, mlp=512),
        hgrn2(2, 160, 40)]), seed=13, page_size=32),
    # one mixer each
    "only_latent": dict(config=model(48, 96, 2.0, 1e-6, [latent(4, 8, 8, 8, 24, 16, mlp=64)]), seed=14, page_size=16),
    "only_hgrn2": dict(config=model(48, 96, 2.0, 1e-6, [hgrn2(3, 8, 12)]), seed=15, page_size=16),
    "only_retention": dict(config=model(48, 96, 0.5, 1e-6, [retention(2, 12, 8, [0.98, 0.999], 12)]), seed=16,
                           page_size=16),
}


def sharpen(config, weights):
    """Makes far tokens matter: query projections of latent attention are scaled up so that
    every softmax falls on one or two keys anywhere in the past; half of the forget gates' lower
    bounds move to 0.999, so that the state still holds the first tokens after hundreds."""
    out = dict(weights)
    for i, e in enumerate(config["layers"]):
        if "weights_of" in e:
            continue
        if e["type"] == "latent_attention":
            out[f"l{i}.mix.uq"] = (weights[f"l{i}.mix.uq"] * 24.0).to(torch.bfloat16).float()
        if e["type"] == "hgrn2":
            low = weights[f"l{i}.mix.lower"].clone()
            low[::2] = 0.999
            out[f"l{i}.mix.lower"] = low.to(torch.bfloat16).float()
    return out


def make_folder(folder, name, sharp=False):
    """Writes config.json and model.safetensors (bfloat16); returns (config, weights as float32)."""
    from dispec_b200.weights import write_safetensors

    spec = CONFIGS[name]
    config = copy.deepcopy(spec["config"])
    weights = plain.random_weights(config, spec["seed"])
    if sharp:
        weights = sharpen(config, weights)
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(config, f)
    write_safetensors(os.path.join(folder, "model.safetensors"),
                      {k: v.to(torch.bfloat16) for k, v in weights.items()})
    return config, weights
