"""Typed configuration of the Ditilix decoder: a stack of layers given one by one, each with one
norm that both of its sublayers read, ``x <- x + r * (mixer(norm(x)) + ff(norm(x)))``.  The
residual stream is kept in float32 and starts as the token's embedding plus a sinusoidal
position vector.  The norm is an RMS norm in groups of consecutive entries.  The mixer is
grouped-query attention without rotation: positions enter through the embedding and through a
query temperature that grows with the logarithm of the position; scores are capped by a tanh;
a layer may read the keys and values that an earlier layer wrote instead of projecting its own.
The feed-forward is a dense layer with a polynomial-of-norms activation, or a mixture of
clamped gated experts whose routing weight multiplies an expert's input, with a gated shared
expert; or absent.

config.json keys::

    architecture     "Ditilix"
    vocab, width     sizes of the embedding table ``embed`` [vocab, width] and the head ``head``
    norm.eps         eps of every norm of the model (layer norms, the last norm, the activation's norms)
    norm.groups      parts of a row with statistics of their own (default 1)
    residual_mult    r, the factor on what a layer adds to the stream (default 1)
    logit_scale      the factor on the logits (default 1)
    layers           a list; entry i has
        type   "attention"
        mixer  heads, kv_heads, dim, vdim, scale; softcap (optional); q_temp {"coef", "every"}
               (optional); kv_from j (optional: no key and value projections, layer j's cache is read)
        mlp    {"kind": "dense", "ff"}, or
               {"kind": "moe", "expert": {"ff", "limit"}, "router": {"experts", "top"},
                "shared": {"ff", "limit"} (optional)}, or null

Tensor names: layer i's start with ``l<i>.``; its norm is ``norm1``, its mixer's tensors
``mix.q / k / v / o``, a dense feed-forward's ``mlp.up / down / act``, a mixture's
``mlp.router``, ``mlp.e<j>.gate / up / down``, ``mlp.shared.gate / up / down / sg``; the model's last
norm is ``final.norm``.

Two constants are the design's own and stand here: the base of the sinusoidal positions and the
slope of the experts' logistic gate; both reach the parts as parameters.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Mapping, Tuple

from .base import ConfigError, LayerSpec, ModelConfig, ModelPlan, PartSpec, ScheduleEntry, _freeze, require

ATTENTION = "attention"
SINUSOID_BASE = 10000.0
EXPERT_GATE_SLOPE = 1.702


def _section(data: Mapping[str, Any], key: str, where: str) -> Mapping[str, Any]:
    value = data.get(key)
    if not isinstance(value, Mapping):
        raise ConfigError(f"config.json: {where}'{key}' must be an object")
    return value


def _int(data: Mapping[str, Any], key: str, where: str, minimum: int = 1) -> int:
    value = data.get(key)
    if isinstance(value, bool) or not isinstance(value, int) or value < minimum:
        raise ConfigError(f"config.json: {where}'{key}' must be an integer >= {minimum}, got {value!r}")
    return value


def _float(data: Mapping[str, Any], key: str, where: str, positive: bool = True) -> float:
    value = data.get(key)
    if isinstance(value, bool) or not isinstance(value, (int, float)) or (positive and not value > 0):
        raise ConfigError(f"config.json: {where}'{key}' must be a {'positive ' if positive else ''}number, got {value!r}")
    return float(value)


@dataclass(frozen=True)
class DitilixConfig(ModelConfig):
    vocab: int
    width: int
    norm_eps: float
    norm_groups: int
    residual_mult: float
    logit_scale: float
    layers: Tuple[Mapping[str, Any], ...]
    max_positions: int = 1 << 20

    architecture = "Ditilix"

    # ------------------------------------------------------------------ reading

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "DitilixConfig":
        layers = data.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        norm = _section(data, "norm", "")
        config = cls(
            vocab=require(data, "vocab", int),
            width=require(data, "width", int),
            norm_eps=_float(norm, "eps", "norm."),
            norm_groups=_int(norm, "groups", "norm.") if norm.get("groups") is not None else 1,
            residual_mult=_float(data, "residual_mult", "", positive=False) if data.get("residual_mult") is not None else 1.0,
            logit_scale=_float(data, "logit_scale", "", positive=False) if data.get("logit_scale") is not None else 1.0,
            layers=tuple(_freeze(dict(layer)) for layer in layers),
            max_positions=int(data.get("max_positions", 1 << 20)),
        )
        config.validate()
        return config

    def validate(self) -> None:
        if self.width % self.norm_groups:
            raise ConfigError(f"config.json: norm.groups {self.norm_groups} does not divide width {self.width}")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]."
            if layer.get("type") != ATTENTION:
                raise ConfigError(f"config.json: {where}'type' must be '{ATTENTION}', got {layer.get('type')!r}")
            mixer = _section(layer, "mixer", where)
            at = where + "mixer."
            heads, kv_heads = _int(mixer, "heads", at), _int(mixer, "kv_heads", at)
            _int(mixer, "dim", at), _int(mixer, "vdim", at), _float(mixer, "scale", at)
            if heads % kv_heads:
                raise ConfigError(f"config.json: {at}heads {heads} is not a multiple of kv_heads {kv_heads}")
            if mixer.get("softcap") is not None:
                _float(mixer, "softcap", at)
            if mixer.get("q_temp") is not None:
                temp = _section(mixer, "q_temp", at)
                _float(temp, "coef", at + "q_temp.", positive=False), _int(temp, "every", at + "q_temp.")
            source = mixer.get("kv_from")
            if source is not None:
                if isinstance(source, bool) or not isinstance(source, int) or not 0 <= source < i:
                    raise ConfigError(f"config.json: {at}kv_from must name an earlier layer, got {source!r}")
                other = self.layers[source]["mixer"]
                if other.get("kv_from") is not None:
                    raise ConfigError(f"config.json: {at}kv_from names layer {source}, which has no keys of its own")
                for key in ("kv_heads", "dim", "vdim"):
                    if other.get(key) != mixer.get(key):
                        raise ConfigError(f"config.json: {at}{key} {mixer.get(key)!r} differs from layer {source}'s "
                                          f"{other.get(key)!r}, whose keys and values this layer reads")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            at = where + "mlp."
            if mlp.get("kind") == "dense":
                _int(mlp, "ff", at)
            elif mlp.get("kind") == "moe":
                expert = _section(mlp, "expert", at)
                _int(expert, "ff", at + "expert."), _float(expert, "limit", at + "expert.")
                router = _section(mlp, "router", at)
                experts, top = _int(router, "experts", at + "router."), _int(router, "top", at + "router.")
                if top > experts:
                    raise ConfigError(f"config.json: {at}router.top {top} exceeds router.experts {experts}")
                if mlp.get("shared") is not None:
                    shared = _section(mlp, "shared", at)
                    _int(shared, "ff", at + "shared."), _float(shared, "limit", at + "shared.")
            else:
                raise ConfigError(f"config.json: {at}kind must be 'dense' or 'moe', got {mlp.get('kind')!r}")

    def to_dict(self) -> dict:
        def thaw(value):
            if isinstance(value, Mapping):
                return {k: thaw(v) for k, v in value.items()}
            if isinstance(value, tuple):
                return [thaw(v) for v in value]
            return value
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.norm_eps, "groups": self.norm_groups}, "residual_mult": self.residual_mult,
                "logit_scale": self.logit_scale, "layers": [thaw(layer) for layer in self.layers]}

    # ------------------------------------------------------------------ the plan

    def _norm(self, name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"size": self.width, "eps": self.norm_eps, "residual": "float32",
                                    "groups": self.norm_groups}, {"weight": name})

    def _mixer(self, layer: Mapping[str, Any], prefix: str) -> PartSpec:
        m = layer["mixer"]
        shared = m.get("kv_from") is not None
        names = [("q_proj", "q"), ("o_proj", "o")] + ([] if shared else [("k_proj", "k"), ("v_proj", "v")])
        temp = m.get("q_temp")
        return PartSpec(
            "attention",
            {"hidden_size": self.width, "n_heads": m["heads"], "n_kv_heads": m["kv_heads"], "head_dim": m["dim"],
             "value_dim": m["vdim"], "scale": float(m["scale"]), "window": None, "chunk": None, "qk_norm_eps": None,
             "prepare": "float32", "softmax_weights": "float32", "position": None,
             "softcap": None if m.get("softcap") is None else float(m["softcap"]),
             "q_temp": None if temp is None else {"coef": float(temp["coef"]), "every": int(temp["every"])},
             "kv": "shared" if shared else "own"},
            {key: f"{prefix}mix.{name}" for key, name in names})

    def _ffn(self, mlp: Mapping[str, Any], prefix: str) -> PartSpec:
        if mlp["kind"] == "dense":
            return PartSpec("polynorm", {"hidden_size": self.width, "intermediate_size": mlp["ff"], "eps": self.norm_eps},
                            {"up_proj": prefix + "mlp.up", "down_proj": prefix + "mlp.down", "act": prefix + "mlp.act"})
        router, shared = mlp["router"], mlp.get("shared")
        tensors: Dict[str, str] = {"router": prefix + "mlp.router"}
        for e in range(router["experts"]):
            for part in ("gate", "up", "down"):
                tensors[f"{part}.{e}"] = f"{prefix}mlp.e{e}.{part}"
        if shared is not None:
            tensors.update(shared_gate_proj=prefix + "mlp.shared.gate", shared_up=prefix + "mlp.shared.up",
                           shared_down=prefix + "mlp.shared.down", shared_gate=prefix + "mlp.shared.sg")
        return PartSpec(
            "routed_clamped_experts",
            {"hidden_size": self.width, "n_experts": router["experts"], "expert_ff": mlp["expert"]["ff"],
             "top": router["top"], "limit": float(mlp["expert"]["limit"]), "slope": EXPERT_GATE_SLOPE,
             "shared_ff": 0 if shared is None else shared["ff"],
             "shared_limit": None if shared is None else float(shared["limit"]), "shared_gated": True},
            tensors)

    def plan(self) -> ModelPlan:
        layers: List[LayerSpec] = []
        schedule: List[ScheduleEntry] = []
        cache_of: Dict[int, int] = {}
        for i, layer in enumerate(self.layers):
            prefix = f"l{i}."
            parts = dict(norm=self._norm(prefix + "norm1"), mixer=self._mixer(layer, prefix), factor=self.residual_mult)
            if layer.get("mlp") is not None:
                parts["ffn"] = self._ffn(layer["mlp"], prefix)
            layers.append(LayerSpec.of("parallel", **parts))
            source = layer["mixer"].get("kv_from")
            if source is None:
                cache_of[i] = len(cache_of)
                schedule.append(ScheduleEntry(layer=i, cache=cache_of[i]))
            else:
                schedule.append(ScheduleEntry(layer=i, cache=cache_of[source], writes_cache=False))
        return ModelPlan(
            hidden_size=self.width,
            vocab_size=self.vocab,
            embedding=PartSpec("embedding", {"vocab_size": self.vocab, "hidden_size": self.width, "stream": "float32",
                                             "positions": {"kind": "sinusoid", "base": SINUSOID_BASE}}, {"weight": "embed"}),
            layers=tuple(layers),
            schedule=tuple(schedule),
            final_norm=self._norm("final.norm"),
            head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": self.width, "tied": False,
                                      "scale": self.logit_scale}, {"weight": "head"}),
            max_positions=self.max_positions,
        )
