"""Typed configuration of the Tidenex decoder: pre-norm layers (layer norms with bias) listed in config.json, each with
one of two mixers and an optional ungated gelu feed-forward; a span of the layers may run several times in a row with
the same weights, the embedding output being added to the stream again before every repeated pass; tied output head.

  "attention"  differential attention: two softmax maps per head over the same values, rotary positions on a part of
               every map (channel i paired with i + dims/2)
  "parallel"   two mixers side by side, each with a weight: softmax attention without rotation (biases, an RMS norm over the
               whole of q and of k, a query temperature, a distance term in the scores) and a gated linear recurrence (HGRN2)

config.json keys: ``architecture`` "Tidenex", ``vocab``, ``width``, ``norm.eps``, ``layers`` (per layer ``type``, ``mixer``
{sizes and constants}, ``mlp`` {``kind`` "dense", ``ff``} or null), optionally ``loop`` {``start``, ``stop``, ``times``} and
``max_positions``.  Tensor names: ``embed``, ``final.norm``(``.b``), per layer ``l<i>.norm1``(``.b``), ``l<i>.norm2``(``.b``),
``l<i>.mix.*`` (``mix.left.*`` / ``mix.right.*`` in a parallel mixer), ``l<i>.mlp.{up,down}``.
"""
import copy
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .base import ConfigError, LayerSpec, ModelPlan, PartSpec, optional, require

MIXERS = ("attention", "parallel")
DEFAULT_MAX_POSITIONS = 1 << 17


def _section(d, key, where):
    v = d.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"config.json: {where}'{key}' must be an object")
    return v


def _heads(m, where, kv=True):
    heads, dim = require(m, "heads", int), require(m, "dim", int)
    vdim = optional(m, "vdim", int, dim)
    if heads <= 0 or dim <= 0 or vdim <= 0:
        raise ConfigError(f"config.json: {where}heads, dim and vdim must be positive")
    if kv:
        g = optional(m, "kv_heads", int, heads)
        if g <= 0 or heads % g:
            raise ConfigError(f"config.json: {where}{heads} heads cannot share {g} kv_heads")


@dataclass(frozen=True)
class TidenexConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    layers: List[Dict[str, Any]] = field(default_factory=list)
    loop: Optional[Dict[str, int]] = None
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
        return len(self.schedule())

    @classmethod
    def from_dict(cls, d, architecture="Tidenex"):
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        loop = d.get("loop")
        if loop is not None:
            loop = {k: require(_section(d, "loop", ""), k, int) for k in ("start", "stop", "times")}
        cfg = cls(architecture=architecture, vocab=require(d, "vocab", int), width=require(d, "width", int),
                  norm_eps=require(_section(d, "norm", ""), "eps", float), layers=copy.deepcopy(layers), loop=loop,
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
            if layer["type"] == "attention":
                _heads(m, where)
                if m.get("rot") is not None:          # a mixer without the key has no rotation
                    rot = _section(m, "rot", where)
                    dims = optional(rot, "dims", int, m["dim"])
                    if dims % 2 or not 0 <= dims <= m["dim"] or not require(rot, "base", float) > 0.0:
                        raise ConfigError(f"config.json: {where}rot.dims must be even and at most dim, rot.base positive")
                require(m, "scale", float)
                if not 0.0 <= require(m, "diff", float) < 1.0:
                    raise ConfigError(f"config.json: {where}diff must lie in [0, 1)")
            else:
                left, right = _section(m, "left", where), _section(m, "right", where)
                _heads(left, where + "left: ")
                _heads(right, where + "right: ", kv=False)
                require(left, "scale", float)
                optional(m, "left_scale", float, 1.0)
                optional(m, "right_scale", float, 1.0)
                if "q_temp" in left and left["q_temp"] is not None:
                    qt = _section(left, "q_temp", where + "left: ")
                    require(qt, "coef", float)
                    if not require(qt, "every", float) > 0.0:
                        raise ConfigError(f"config.json: {where}left: q_temp.every must be positive")
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or optional(mlp, "kind", str, "dense") != "dense":
                    raise ConfigError(f"config.json: {where}mlp.kind must be 'dense' (or mlp null)")
                if require(mlp, "ff", int) <= 0:
                    raise ConfigError(f"config.json: {where}mlp.ff must be positive")
        if self.loop is not None:
            a, b, times = self.loop["start"], self.loop["stop"], self.loop["times"]
            if not 0 <= a < b <= len(self.layers) or times < 1:
                raise ConfigError("config.json: loop needs 0 <= start < stop <= number of layers and times >= 1")

    def to_dict(self):
        d = {"architecture": self.architecture, "layers": copy.deepcopy(self.layers), "norm": {"eps": self.norm_eps},
             "vocab": self.vocab, "width": self.width}
        if self.loop is not None:
            d["loop"] = dict(self.loop)
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_positions
        if self.eos_token_id is not None:
            d["eos_token_id"] = self.eos_token_id
        return d

    def schedule(self):
        """(order in which the layers run, positions of that order at which a repeated pass starts)."""
        n = len(self.layers)
        if self.loop is None:
            return list(range(n)), ()
        a, b, times = self.loop["start"], self.loop["stop"], self.loop["times"]
        order, again = list(range(a)), []
        for p in range(times):
            if p > 0:
                again.append(len(order))
            order += list(range(a, b))
        return order + list(range(b, n)), tuple(again)

    def _mixer(self, layer):
        m, W, eps = layer["mixer"], self.width, self.norm_eps
        if layer["type"] == "attention":
            dim = m["dim"]
            rot = m.get("rot") or {"dims": 0, "base": 10000.0}
            return PartSpec("differential_attention", {
                "hidden_size": W, "num_heads": m["heads"], "num_kv_heads": m.get("kv_heads", m["heads"]), "head_dim": dim,
                "v_head_dim": m.get("vdim", dim), "scale": float(m["scale"]), "diff": float(m["diff"]), "eps": eps,
                "position": PartSpec("rope_halves", {"head_dim": dim, "rotary_dims": rot.get("dims", dim), "theta": float(rot["base"])})})
        left, right = m["left"], m["right"]
        qt = left.get("q_temp") or {}
        return PartSpec("side_by_side", {"mixers": [
            PartSpec("distance_attention", {
                "hidden_size": W, "num_heads": left["heads"], "num_kv_heads": left.get("kv_heads", left["heads"]),
                "head_dim": left["dim"], "v_head_dim": left.get("vdim", left["dim"]), "scale": float(left["scale"]), "eps": eps,
                "temp_coef": float(qt.get("coef", 0.0)), "temp_every": float(qt.get("every", 0.0)),
                "out_scale": float(m.get("left_scale", 1.0)), "prefix": "mix.left."}),
            PartSpec("gated_write", {
                "hidden_size": W, "num_heads": right["heads"], "head_dim": right["dim"], "v_head_dim": right.get("vdim", right["dim"]),
                "eps": eps, "out_scale": float(m.get("right_scale", 1.0)), "prefix": "mix.right."})]})

    def plan(self) -> ModelPlan:
        W = self.width

        def norm(name):
            return PartSpec("layernorm", {"size": W, "eps": self.norm_eps, "names": {"weight": name, "bias": name + ".b"}})
        layers = []
        for i, layer in enumerate(self.layers):
            mlp = layer.get("mlp")
            ff = PartSpec("none", {}) if mlp is None else PartSpec("dense", {
                "hidden_size": W, "intermediate_size": mlp["ff"], "activation": "gelu", "names": {"up": "mlp.up", "down": "mlp.down"}})
            layers.append(LayerSpec(block="pre_norm", mixer=self._mixer(layer), feed_forward=ff,
                                    norms={"input": norm("norm1"), "post_mixer": None if mlp is None else norm("norm2")},
                                    weight_prefix=f"l{i}.", norm_prefixes={"input": "", "post_mixer": ""}))
        order, again = self.schedule()
        return ModelPlan(
            hidden_size=W, vocab_size=self.vocab, max_positions=self.max_positions,
            embedding=PartSpec("embedding", {"vocab_size": self.vocab, "hidden_size": W, "names": {"weight": "embed"}}),
            final_norm=norm("final.norm"),
            lm_head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": W, "tied": True, "names": {"weight": "head"}}),
            layers=layers, schedule=order, embedding_prefix="", final_norm_prefix="", lm_head_prefix="",
            add_embedding_before=again)
