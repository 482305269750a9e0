"""Puludra: a decoder whose layers are listed one by one in config.json, each with a mixer of
its own kind (latent attention, HGRN2, retention), an optional dense xIELU feed-forward, and the
norm after the sum (x <- norm(alpha * x + sublayer(x))).  A layer may run another layer's
weights (``weights_of``) with a cache and state of its own.

config.json: ``architecture``, ``vocab``, ``width``, ``postln_alpha``, ``norm.eps`` and ``layers``:
a list of {``type``, ``mixer``: sizes and constants of the mixer, ``mlp``: {``kind``, ``ff``} or null,
``weights_of``: index (optional)}.  Tensors: ``embed``, ``head``, ``final.norm`` and, for layer i,
``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``; matrices are stored [out, in].
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import ClassVar

from dispec_b200.config.model_config import ConfigError, ModelConfig, _require
from dispec_b200.models.spec import LayerCall, ModelSpec
from dispec_b200.parts.base import PartSpec
from dispec_b200.registry import register_architecture

_MIXER_KEYS = {
    "latent_attention": ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank", "scale", "rot"),
    "hgrn2": ("heads", "dim", "vdim"),
    "retention": ("heads", "dim", "vdim", "decay", "rot"),
}


@dataclass(frozen=True)
class PuludraConfig(ModelConfig):
    architecture: ClassVar[str] = "Puludra"

    vocab_size: int
    hidden_size: int
    alpha: float
    eps: float
    layers: tuple  # of dict, as in config.json (deep copies; never mutated)
    max_position_embeddings: int = 0  # 0: no limit of the model's own

    @classmethod
    def from_dict(cls, d: dict) -> "PuludraConfig":
        where = cls.architecture
        _require(d, ["vocab", "width", "postln_alpha", "norm", "layers"], where)
        _require(d["norm"], ["eps"], where + " norm")
        layers = []
        if not isinstance(d["layers"], list) or not d["layers"]:
            raise ConfigError(f"{where}: 'layers' must be a non-empty list")
        for i, e in enumerate(d["layers"]):
            at = f"{where} layers[{i}]"
            _require(e, ["type", "mixer"], at)
            if e["type"] not in _MIXER_KEYS:
                raise ConfigError(f"{at}: mixer type {e['type']!r} is not implemented "
                                  f"(known: {', '.join(sorted(_MIXER_KEYS))})")
            _require(e["mixer"], list(_MIXER_KEYS[e["type"]]), at + " mixer")
            m = e["mixer"]
            if "rot" in _MIXER_KEYS[e["type"]]:
                _require(m["rot"], ["base", "dims"], at + " mixer.rot")
                limit = m["rot_dim"] if e["type"] == "latent_attention" else m["dim"]
                if m["rot"]["dims"] % 2 or not 0 <= m["rot"]["dims"] <= limit:
                    raise ConfigError(f"{at}: rot.dims={m['rot']['dims']} must be even and at most {limit}")
            if e["type"] == "retention" and len(m["decay"]) != m["heads"]:
                raise ConfigError(f"{at}: {len(m['decay'])} decays for {m['heads']} heads")
            mlp = e.get("mlp")
            if mlp is not None:
                _require(mlp, ["kind", "ff"], at + " mlp")
                if mlp["kind"] != "dense":
                    raise ConfigError(f"{at}: mlp.kind={mlp['kind']!r} is not implemented (only 'dense')")
            j = e.get("weights_of")
            if j is not None and not (isinstance(j, int) and 0 <= j < len(d["layers"]) and j != i):
                raise ConfigError(f"{at}: weights_of={j!r} is not the index of another layer")
            layers.append(copy.deepcopy(e))
        cfg = cls(vocab_size=int(d["vocab"]), hidden_size=int(d["width"]), alpha=float(d["postln_alpha"]),
                  eps=float(d["norm"]["eps"]), layers=tuple(layers),
                  max_position_embeddings=int(d.get("max_position_embeddings", 0)))
        for i in range(len(layers)):
            cfg.weights_layer(i)  # raises on a cycle
        return cfg

    def weights_layer(self, i: int) -> int:
        """Index of the layer whose tensors layer i runs (i itself unless it names another)."""
        seen = {i}
        while self.layers[i].get("weights_of") is not None:
            i = self.layers[i]["weights_of"]
            if i in seen:
                raise ConfigError(f"{self.architecture}: 'weights_of' runs in a circle at layer {i}")
            seen.add(i)
        return i

    def to_dict(self) -> dict:
        d = {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
             "postln_alpha": self.alpha, "norm": {"eps": self.eps}, "layers": copy.deepcopy(list(self.layers))}
        if self.max_position_embeddings:
            d["max_position_embeddings"] = self.max_position_embeddings
        return d

    def flat(self) -> dict:
        out = super().flat()
        out["num_layers"] = len(self.layers)
        out["layer_types"] = ",".join(e["type"] for e in self.layers)
        return out


def _mixer_spec(cfg: PuludraConfig, kind: str, m: dict, prefix: str) -> PartSpec:
    h = cfg.hidden_size
    t = lambda *names: {(n if "." in n or n == "lower" else n + ".weight"): prefix + n for n in names}
    if kind == "retention":
        rotary = PartSpec("position_encoding", "rotary", {"head_dim": m["dim"], "theta": m["rot"]["base"],
                                                          "rotary_dim": m["rot"]["dims"], "layout": "halves"})
        if not m["rot"]["dims"]:
            rotary = PartSpec("position_encoding", "none")
        return PartSpec("mixer", "retention",
                        {"hidden_size": h, "num_heads": m["heads"], "dim": m["dim"], "vdim": m["vdim"],
                         "decay": tuple(m["decay"]), "eps": cfg.eps, "position_encoding": rotary},
                        t("q", "k", "v", "g", "o"))
    if kind == "hgrn2":
        names = t("q", "f", "v", "o")
        names.update({"f.bias": prefix + "f.b", "lower": prefix + "lower", "norm.weight": prefix + "norm"})
        return PartSpec("mixer", "hgrn2", {"hidden_size": h, "num_heads": m["heads"], "dim": m["dim"],
                                           "vdim": m["vdim"], "eps": cfg.eps}, names)
    rotary = PartSpec("position_encoding", "rotary", {"head_dim": m["rot_dim"], "theta": m["rot"]["base"],
                                                      "rotary_dim": m["rot"]["dims"], "layout": "interleaved"})
    if not m["rot"]["dims"]:
        rotary = PartSpec("position_encoding", "none")
    names = {f"{n}.weight": prefix + n for n in ("dq", "uq", "dkv", "uk", "uv", "o")}
    names.update({"dq.norm": prefix + "dq.norm", "dkv.norm": prefix + "dkv.norm"})
    return PartSpec("mixer", "latent_attention",
                    {"hidden_size": h, "num_heads": m["heads"], "dim": m["dim"], "rot_dim": m["rot_dim"],
                     "vdim": m["vdim"], "kv_rank": m["kv_rank"], "q_rank": m["q_rank"], "scale": m["scale"],
                     "eps": cfg.eps, "position_encoding": rotary}, names)


def build_puludra(cfg: PuludraConfig) -> ModelSpec:
    h = cfg.hidden_size
    norm = lambda name: PartSpec("norm", "rms_norm_f32", {"hidden_size": h, "eps": cfg.eps}, {"weight": name})
    blocks, index_of, schedule = [], {}, []
    for i in range(len(cfg.layers)):
        src = cfg.weights_layer(i)
        if src not in index_of:
            e, p = cfg.layers[src], f"l{src}."
            params = {"mixer_norm": norm(p + "norm1"), "mixer": _mixer_spec(cfg, e["type"], e["mixer"], p + "mix."),
                      "alpha": cfg.alpha}
            if e.get("mlp") is not None:
                params["ffn_norm"] = norm(p + "norm2")
                params["feed_forward"] = PartSpec(
                    "feed_forward", "xielu", {"hidden_size": h, "intermediate_size": e["mlp"]["ff"]},
                    {"up.weight": p + "mlp.up", "down.weight": p + "mlp.down", "act": p + "mlp.act"})
            index_of[src] = len(blocks)
            blocks.append(PartSpec("block", "post_norm", params))
        schedule.append(LayerCall(index_of[src], i, True))
    return ModelSpec(
        architecture=cfg.architecture,
        embedding=PartSpec("embedding", "token_embedding", {"vocab_size": cfg.vocab_size, "hidden_size": h},
                           {"weight": "embed"}),
        layers=blocks, final_norm=norm("final.norm"),
        head=PartSpec("head", "linear_head", {"vocab_size": cfg.vocab_size, "hidden_size": h}, {"weight": "head"}),
        schedule=schedule, vocab_size=cfg.vocab_size, max_position=cfg.max_position_embeddings)


register_architecture(PuludraConfig.architecture, PuludraConfig, build_puludra)
