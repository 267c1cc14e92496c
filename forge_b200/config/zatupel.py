"""Typed configuration of the Zatupel decoder: a list of layers, each with one of three mixers (attention over a window
with kept first tokens whose heads exchange weights; a decay-and-bonus state mixer; a generalized-delta-rule state
mixer) and an optional gated feed-forward, both branches reading the same residual stream through norms of their own.

config.json keys: ``architecture`` "Zatupel", ``vocab``, ``width``, ``embedding.scale``, ``norm.eps``, ``layers`` (per
layer ``type``, ``mixer`` {sizes and constants of the mixer}, ``mlp`` {``kind`` "dense", ``ff``} or null), and optionally
``max_positions`` (how far a sequence may grow; nothing in the design limits it).  Tensor names: ``embed``, ``head``,
``final.norm``, and per layer ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.{gate,up,down}``.
"""
import copy
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .base import ConfigError, LayerSpec, ModelPlan, PartSpec, coerce, optional, require

MIXERS = ("attention", "wkv", "general_delta")
DEFAULT_MAX_POSITIONS = 1 << 17


def _section(d, key, where):
    v = d.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"config.json: {where}'{key}' must be an object")
    return v


@dataclass(frozen=True)
class ZatupelConfig:
    architecture: str
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    layers: List[Dict[str, Any]] = field(default_factory=list)
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_id: Optional[int] = None

    # what the command line and the benchmark ask any configuration
    @property
    def vocab_size(self):
        return self.vocab

    @property
    def hidden_size(self):
        return self.width

    @property
    def num_hidden_layers(self):
        return len(self.layers)

    @classmethod
    def from_dict(cls, d, architecture="Zatupel"):
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        cfg = cls(architecture=architecture, vocab=require(d, "vocab", int), width=require(d, "width", int),
                  embedding_scale=optional(_section(d, "embedding", ""), "scale", float, 1.0) if "embedding" in d else 1.0,
                  norm_eps=require(_section(d, "norm", ""), "eps", float), layers=copy.deepcopy(layers),
                  max_positions=optional(d, "max_positions", int, DEFAULT_MAX_POSITIONS),
                  eos_token_id=optional(d, "eos_token_id", int, None))
        cfg.validate()
        return cfg

    def validate(self):
        if self.vocab <= 0 or self.width <= 0 or self.max_positions <= 0 or not self.norm_eps > 0.0:
            raise ConfigError("config.json: vocab, width, max_positions and norm.eps must be positive")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]: "
            if not isinstance(layer, dict) or layer.get("type") not in MIXERS:
                raise ConfigError(f"config.json: {where}'type' must be one of {MIXERS}")
            m = _section(layer, "mixer", where)
            heads, dim = require(m, "heads", int), require(m, "dim", int)
            if heads <= 0 or dim <= 0:
                raise ConfigError(f"config.json: {where}heads and dim must be positive")
            if layer["type"] == "attention":
                kv = optional(m, "kv_heads", int, heads)
                if kv <= 0 or heads % kv:
                    raise ConfigError(f"config.json: {where}{heads} heads cannot share {kv} kv_heads")
                mask, rot = _section(m, "mask", where), _section(m, "rot", where)
                if require(mask, "size", int) <= 0 or optional(mask, "keep_first", int, 0) < 0:
                    raise ConfigError(f"config.json: {where}mask.size must be positive and mask.keep_first not negative")
                dims = optional(rot, "dims", int, dim)
                if dims % 2 or not 0 <= dims <= dim or not require(rot, "base", float) > 0.0:
                    raise ConfigError(f"config.json: {where}rot.dims must be even and at most dim, rot.base positive")
                require(m, "scale", float)
                optional(m, "v_mix", bool, False)
                if optional(m, "vdim", int, dim) <= 0:
                    raise ConfigError(f"config.json: {where}vdim must be positive")
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or optional(mlp, "kind", str, "dense") != "dense":
                    raise ConfigError(f"config.json: {where}mlp.kind must be 'dense' (or mlp null)")
                if require(mlp, "ff", int) <= 0:
                    raise ConfigError(f"config.json: {where}mlp.ff must be positive")

    def to_dict(self):
        d = {"architecture": self.architecture, "embedding": {"scale": self.embedding_scale}, "layers": copy.deepcopy(self.layers),
             "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width}
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_positions
        if self.eos_token_id is not None:
            d["eos_token_id"] = self.eos_token_id
        return d

    def _mixer(self, i, layer, first_blend):
        m, W = layer["mixer"], self.width
        if layer["type"] == "attention":
            dim = m["dim"]
            blend = bool(m.get("v_mix", False))
            return PartSpec("headmix_attention", {
                "hidden_size": W, "num_heads": m["heads"], "num_kv_heads": m.get("kv_heads", m["heads"]), "head_dim": dim,
                "v_head_dim": m.get("vdim", dim), "scale": float(m["scale"]), "window": m["mask"]["size"],
                "keep_first": m["mask"].get("keep_first", 0), "head_mix": True, "head_gate": True,
                "value_mix": None if not blend else ("source" if i == first_blend else "blend"),
                "position": PartSpec("rope_pairs", {"head_dim": dim, "rotary_dims": m["rot"].get("dims", dim),
                                                    "theta": float(m["rot"]["base"])})})
        params = {"hidden_size": W, "num_heads": m["heads"], "head_dim": m["dim"], "eps": self.norm_eps}
        if "rank" in m:                      # only random weights need it: a file's tensors say it themselves
            params["rank"] = coerce("rank", m["rank"], int)
        return PartSpec(layer["type"], params)

    def plan(self) -> ModelPlan:
        W = self.width

        def norm(name):
            return PartSpec("rmsnorm", {"size": W, "eps": self.norm_eps, "names": {"weight": name}})
        blends = [i for i, layer in enumerate(self.layers) if layer["type"] == "attention" and layer["mixer"].get("v_mix", False)]
        first_blend = blends[0] if blends else None
        layers = []
        for i, layer in enumerate(self.layers):
            mlp = layer.get("mlp")
            ff = PartSpec("none", {}) if mlp is None else PartSpec("geglu", {
                "hidden_size": W, "intermediate_size": mlp["ff"], "suffix": "",
                "names": {"gate": "mlp.gate", "up": "mlp.up", "down": "mlp.down"}})
            layers.append(LayerSpec(block="parallel", mixer=self._mixer(i, layer, first_blend), feed_forward=ff,
                                    norms={"mixer": norm("norm1"), "feed_forward": None if mlp is None else norm("norm2")},
                                    weight_prefix=f"l{i}."))
        return ModelPlan(
            hidden_size=W, vocab_size=self.vocab, max_positions=self.max_positions,
            embedding=PartSpec("embedding", {"vocab_size": self.vocab, "hidden_size": W, "scale": self.embedding_scale,
                                             "names": {"weight": "embed"}}),
            final_norm=norm("final.norm"),
            lm_head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": W, "tied": False, "names": {"weight": "head"}}),
            layers=layers, schedule=list(range(len(layers))), embedding_prefix="", final_norm_prefix="", lm_head_prefix="")
