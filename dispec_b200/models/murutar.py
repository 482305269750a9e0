"""Murutar: a decoder whose layers are listed one by one in config.json, each with a mixer
(``attention``: grouped-query attention with a sliding window, a sink in the softmax, partial
rotation and values blended with the first such layer's; ``lightning``: linear attention with a
fixed decay per head) and an optional feed-forward (``dense``: a clamped gated unit; ``moe``:
experts with grouped routing).  Pre-norm layer norms without bias, every sublayer's result
scaled per channel and gated before the 32-bit residual sum, a per-layer input from a token
table after the feed-forward, and a tied output matrix with squashed logits.

config.json: ``architecture``, ``vocab``, ``width``, ``embedding.scale``, ``norm.eps``,
``logit_softcap`` (optional), ``token_side.dim`` (optional) and ``layers``: a list of {``type``,
``mixer``: sizes and constants of the mixer, ``mlp``: {``kind``, ...} or null}.  Tensors: ``embed``,
``side.embed``, ``final.norm`` and, for layer i, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.ls1|2``,
``l<i>.rg1|2`` (+ ``.b``), ``l<i>.mix.*``, ``l<i>.mlp.*``, ``l<i>.side.*``; matrices are stored [out, in].
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import ClassVar

from dispec_b200.config.model_config import ConfigError, ModelConfig, _require
from dispec_b200.models.spec import ModelSpec
from dispec_b200.parts.base import PartSpec
from dispec_b200.registry import register_architecture

_MIXER_KEYS = {
    "attention": ("heads", "kv_heads", "dim", "vdim", "scale"),
    "lightning": ("heads", "dim", "vdim", "decay"),
}


def _window(m: dict) -> int:
    return int((m.get("mask") or {}).get("size") or 0)


def _rot(m: dict) -> tuple[int, float]:
    rot = m.get("rot") or {}
    return int(rot.get("dims") or 0), float(rot.get("base") or 1.0)


@dataclass(frozen=True)
class MurutarConfig(ModelConfig):
    architecture: ClassVar[str] = "Murutar"

    vocab_size: int
    hidden_size: int
    embedding_scale: float
    eps: float
    logit_softcap: float  # 0: logits are not squashed
    token_side_dim: int  # 0: no per-layer token input
    layers: tuple  # of dict, as in config.json (deep copies; never mutated)
    max_position_embeddings: int = 0  # 0: no limit of the model's own

    @classmethod
    def from_dict(cls, d: dict) -> "MurutarConfig":
        where = cls.architecture
        _require(d, ["vocab", "width", "norm", "layers"], where)
        _require(d["norm"], ["eps"], where + " norm")
        if not isinstance(d["layers"], list) or not d["layers"]:
            raise ConfigError(f"{where}: 'layers' must be a non-empty list")
        layers, mixed_width = [], None
        for i, e in enumerate(d["layers"]):
            at = f"{where} layers[{i}]"
            _require(e, ["type", "mixer"], at)
            if e["type"] not in _MIXER_KEYS:
                raise ConfigError(f"{at}: mixer type {e['type']!r} is not implemented "
                                  f"(known: {', '.join(sorted(_MIXER_KEYS))})")
            m = e["mixer"]
            _require(m, list(_MIXER_KEYS[e["type"]]), at + " mixer")
            if e["type"] == "attention":
                if m["heads"] % m["kv_heads"]:
                    raise ConfigError(f"{at}: heads={m['heads']} is not a multiple of kv_heads={m['kv_heads']}")
                dims, base = _rot(m)
                if dims and (dims % 2 or dims > m["dim"] or not base > 0):
                    raise ConfigError(f"{at}: rot.dims={dims} must be even and at most dim={m['dim']}, rot.base positive")
                if _window(m) < 0:
                    raise ConfigError(f"{at}: mask.size must not be negative")
                if m.get("v_mix"):
                    width = (m["kv_heads"], m["vdim"])
                    if mixed_width is not None and width != mixed_width:
                        raise ConfigError(f"{at}: v_mix layers must agree in (kv_heads, vdim): {width} vs {mixed_width}")
                    mixed_width = width
            elif len(m["decay"]) != m["heads"]:
                raise ConfigError(f"{at}: {len(m['decay'])} decays for {m['heads']} heads")
            mlp = e.get("mlp")
            if mlp is not None:
                _require(mlp, ["kind"], at + " mlp")
                if mlp["kind"] == "dense":
                    _require(mlp, ["ff", "limit"], at + " mlp")
                elif mlp["kind"] == "moe":
                    _require(mlp, ["expert", "router"], at + " mlp")
                    _require(mlp["expert"], ["ff"], at + " mlp.expert")
                    _require(mlp["router"], ["experts", "top"], at + " mlp.router")
                else:
                    raise ConfigError(f"{at}: mlp.kind={mlp['kind']!r} is not implemented (known: dense, moe)")
            layers.append(copy.deepcopy(e))
        side = d.get("token_side") or {}
        return cls(vocab_size=int(d["vocab"]), hidden_size=int(d["width"]),
                   embedding_scale=float((d.get("embedding") or {}).get("scale", 1.0)),
                   eps=float(d["norm"]["eps"]), logit_softcap=float(d.get("logit_softcap") or 0.0),
                   token_side_dim=int(side.get("dim") or 0), layers=tuple(layers),
                   max_position_embeddings=int(d.get("max_position_embeddings", 0)))

    def to_dict(self) -> dict:
        d = {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
             "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.eps},
             "layers": copy.deepcopy(list(self.layers))}
        if self.logit_softcap:
            d["logit_softcap"] = self.logit_softcap
        if self.token_side_dim:
            d["token_side"] = {"dim": self.token_side_dim}
        if self.max_position_embeddings:
            d["max_position_embeddings"] = self.max_position_embeddings
        return d

    def flat(self) -> dict:
        out = super().flat()
        out["num_layers"] = len(self.layers)
        out["layer_types"] = ",".join(e["type"] for e in self.layers)
        return out


def _mixer_spec(cfg: MurutarConfig, e: dict, prefix: str, mix_role) -> PartSpec:
    h, m = cfg.hidden_size, e["mixer"]
    names = lambda *ns: {n + ".weight": prefix + n for n in ns}
    if e["type"] == "lightning":
        return PartSpec("mixer", "lightning",
                        {"hidden_size": h, "num_heads": m["heads"], "dim": m["dim"], "vdim": m["vdim"],
                         "decay": tuple(m["decay"]), "eps": cfg.eps}, names("q", "k", "v", "g", "o", "norm"))
    dims, base = _rot(m)
    rotary = PartSpec("position_encoding", "none")
    if dims:
        rotary = PartSpec("position_encoding", "rotary", {"head_dim": m["dim"], "theta": base, "rotary_dim": dims,
                                                          "layout": "halves", "exact_table": True})
    tensors = names("q", "k", "v", "o")
    if mix_role is not None:
        tensors["value_mix"] = prefix + "vmix"
    return PartSpec("mixer", "sink_attention",
                    {"hidden_size": h, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "key_dim": m["dim"],
                     "value_dim": m["vdim"], "scale": m["scale"], "window": _window(m), "sink": True,
                     "position_encoding": rotary, "value_mix": mix_role}, tensors)


def _ffn_spec(cfg: MurutarConfig, mlp: dict, prefix: str) -> PartSpec:
    h = cfg.hidden_size
    if mlp["kind"] == "dense":
        return PartSpec("feed_forward", "clamped_glu",
                        {"hidden_size": h, "intermediate_size": mlp["ff"], "limit": mlp["limit"]},
                        {n + ".weight": prefix + n for n in ("gate", "up", "down")})
    r = mlp["router"]
    groups = r.get("groups") or {}
    E = int(r["experts"])
    tensors = {"router.weight": prefix + "router"}
    for i in range(E):
        tensors[f"experts.{i}.up.weight"] = f"{prefix}e{i}.up"
        tensors[f"experts.{i}.down.weight"] = f"{prefix}e{i}.down"
    return PartSpec("feed_forward", "grouped_moe",
                    {"hidden_size": h, "intermediate_size": mlp["expert"]["ff"], "num_experts": E, "top": int(r["top"]),
                     "num_groups": int(groups.get("count") or 1),
                     "keep_groups": int(groups.get("keep") or groups.get("count") or 1)}, tensors)


def build_murutar(cfg: MurutarConfig) -> ModelSpec:
    h, L = cfg.hidden_size, len(cfg.layers)
    norm = lambda name: PartSpec("norm", "layer_norm_f32", {"hidden_size": h, "eps": cfg.eps}, {"weight": name})
    blocks, seen_mix = [], False
    for i, e in enumerate(cfg.layers):
        p = f"l{i}."
        mix_role = None
        if e["type"] == "attention" and e["mixer"].get("v_mix"):
            mix_role = ("blend" if seen_mix else "source", "v")
            seen_mix = True
        params = {"hidden_size": h, "mixer_norm": norm(p + "norm1"), "mixer": _mixer_spec(cfg, e, p + "mix.", mix_role)}
        tensors = {"scale1": p + "ls1", "gate1.weight": p + "rg1", "gate1.bias": p + "rg1.b"}
        if e.get("mlp") is not None:
            params["ffn_norm"] = norm(p + "norm2")
            params["feed_forward"] = _ffn_spec(cfg, e["mlp"], p + "mlp.")
            tensors.update({"scale2": p + "ls2", "gate2.weight": p + "rg2", "gate2.bias": p + "rg2.b"})
        if cfg.token_side_dim:
            d = cfg.token_side_dim
            params["token_input"] = PartSpec(
                "feed_forward", "token_table_input",
                {"hidden_size": h, "vocab_size": cfg.vocab_size, "table_width": L * d, "offset": i * d, "dim": d,
                 "eps": cfg.eps},
                {"table": "side.embed", "gate.weight": p + "side.gate", "proj.weight": p + "side.proj",
                 "norm.weight": p + "side.norm"})
        blocks.append(PartSpec("block", "gated_pre_norm", params, tensors))
    return ModelSpec(
        architecture=cfg.architecture,
        embedding=PartSpec("embedding", "scaled_embedding",
                           {"vocab_size": cfg.vocab_size, "hidden_size": h, "scale": cfg.embedding_scale},
                           {"weight": "embed"}),
        layers=blocks, final_norm=norm("final.norm"),
        head=PartSpec("head", "linear_head", {"vocab_size": cfg.vocab_size, "hidden_size": h,
                                              "softcap": cfg.logit_softcap or None}, {"weight": "embed"}),
        schedule=[], vocab_size=cfg.vocab_size, max_position=cfg.max_position_embeddings)


register_architecture(MurutarConfig.architecture, MurutarConfig, build_murutar)
