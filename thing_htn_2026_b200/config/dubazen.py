"""Typed configuration of the Dubazen decoder: a stack of layers given one by one over a residual
stream of several copies joined by hyper-connections, each layer with a token mixer of one of three
kinds and an optional mixture-of-experts feed-forward.

The stream is ``streams`` copies in float32, all equal to the token's embedding times
``embedding.scale`` at the start.  A sublayer reads a weighted sum of the copies through an RMS
norm whose gain is one number, and its output is added to every copy with a weight of its own
while the copies are remixed (block ``hyper_connections``); without ``streams`` the model has one
plain stream, ``x <- x + f(norm(x))``.  The model ends with the norm of the copies' sum and the head.

config.json keys::

    architecture      "Dubazen"
    vocab, width      sizes of the embedding table ``embed`` [vocab, width] and the head ``head``
    embedding.scale   the factor on the embedding (default 1)
    norm.eps          eps of every norm of the model
    streams           copies of the residual stream (absent: one plain stream, no hyper-connection tensors)
    layers            a list; entry i has
        type   "parallel", "gla" or "mamba1"
        mixer  the mixer's sizes and constants, see below
        mlp    {"kind": "moe", "expert": {"ff", "limit"}, "router": {"experts", "top"},
                "shared": {"ff", "limit"} (optional)} or null (no feed-forward in this layer)

    mixer of "parallel":  left {heads, kv_heads, dim, vdim, scale, rot {"base", "dims"}}: softmax attention with
                          biased projections, rotation of the first rot.dims entries of a head (entry i paired with
                          i + dims/2), unit-RMS queries and keys, values turned by their position over all vdim
                          entries, a sink per head and a logistic output gate;
                          right {heads, dim, vdim, decay [heads]}: linear attention on silu'd projections with one
                          constant decay per head, one RMS norm over all heads, a logistic gate;
                          left_scale, right_scale: the weights of their sum.
    mixer of "gla":       heads, dim, vdim, tau: linear attention with a decay per key channel
                          ``logistic(z)^(1/tau)``, z through a low-rank pair of projections; RMS norm per head,
                          a silu gate.  ``rank`` (optional): the channels between the two projections; without it the
                          shapes of the checkpoint's two tensors give it (random weights need it).
    mixer of "mamba1":    inner, state, dt_rank, conv: the selective scan behind a short causal convolution.

Tensor names: layer i's start with ``l<i>.``; its norms are ``norm1`` and ``norm2`` (one number each), its
hyper-connections ``hc1.in / mix / out`` (mixer) and ``hc2.*`` (feed-forward), its mixer's tensors
``mix.*`` (``mix.left.*`` and ``mix.right.*`` for "parallel"; a bias is its weight's name with ``.b``), its
feed-forward's ``mlp.router``, ``mlp.e<j>.gate / up / down``, ``mlp.shared.gate / up / down``; the model's last norm
is ``final.norm``.

Constants of the design stand here and reach the parts as parameters: the slope 1.702 of the experts'
logistic gate, the 1e-20 added to the sum of the chosen experts' scores, and the ``dim^-1/2`` on the
queries of "gla".
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, List, Mapping, Optional, Tuple

from .base import ConfigError, LayerSpec, ModelConfig, ModelPlan, PartSpec, ScheduleEntry, _freeze, require

PARALLEL = "parallel"
GLA = "gla"
MAMBA = "mamba1"

EXPERT_GATE_SLOPE = 1.702
ROUTER_SUM_FLOOR = 1e-20
MAX_STREAMS = 16


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
class DubazenConfig(ModelConfig):
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    streams: Optional[int]
    layers: Tuple[Mapping[str, Any], ...]
    max_positions: int = 1 << 20

    architecture = "Dubazen"

    # ------------------------------------------------------------------ reading

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "DubazenConfig":
        layers = data.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        embedding = data.get("embedding") or {}
        config = cls(
            vocab=require(data, "vocab", int),
            width=require(data, "width", int),
            embedding_scale=_float(embedding, "scale", "embedding.") if "scale" in embedding else 1.0,
            norm_eps=_float(_section(data, "norm", ""), "eps", "norm."),
            streams=None if data.get("streams") is None else _int(data, "streams", ""),
            layers=tuple(_freeze(dict(layer)) for layer in layers),
            max_positions=int(data.get("max_positions", 1 << 20)),
        )
        config.validate()
        return config

    def validate(self) -> None:
        if self.streams is not None and self.streams > MAX_STREAMS:
            raise ConfigError(f"config.json: 'streams' {self.streams} is more than the {MAX_STREAMS} this library runs")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]."
            kind = layer.get("type")
            if kind not in (PARALLEL, GLA, MAMBA):
                raise ConfigError(f"config.json: {where}'type' must be '{PARALLEL}', '{GLA}' or '{MAMBA}', got {kind!r}")
            mixer = _section(layer, "mixer", where)
            at = where + "mixer."
            if kind == PARALLEL:
                left, right = _section(mixer, "left", at), _section(mixer, "right", at)
                heads, kv_heads = _int(left, "heads", at + "left."), _int(left, "kv_heads", at + "left.")
                dim, vdim = _int(left, "dim", at + "left."), _int(left, "vdim", at + "left.")
                if heads % kv_heads:
                    raise ConfigError(f"config.json: {at}left.heads {heads} is not a multiple of kv_heads {kv_heads}")
                if vdim % 2:
                    raise ConfigError(f"config.json: {at}left.vdim {vdim} must be even (the values turn in pairs)")
                _float(left, "scale", at + "left.")
                rot = _section(left, "rot", at + "left.")
                dims = _int(rot, "dims", at + "left.rot.", 0)
                if dims % 2 or dims > dim:
                    raise ConfigError(f"config.json: {at}left.rot.dims {dims} must be even and at most {dim}")
                _float(rot, "base", at + "left.rot.")
                for key in ("mask", "window"):
                    if left.get(key) is not None:
                        raise ConfigError(f"config.json: {at}left.{key}: this mixer sees every earlier position")
                r_heads = _int(right, "heads", at + "right.")
                _int(right, "dim", at + "right.")
                _int(right, "vdim", at + "right.")
                decay = right.get("decay")
                if not isinstance(decay, (list, tuple)) or len(decay) != r_heads \
                        or any(isinstance(v, bool) or not isinstance(v, (int, float)) for v in decay):
                    raise ConfigError(f"config.json: {at}right.decay must be a list of {r_heads} numbers")
                _float(mixer, "left_scale", at, positive=False)
                _float(mixer, "right_scale", at, positive=False)
            elif kind == GLA:
                _int(mixer, "heads", at), _int(mixer, "dim", at), _int(mixer, "vdim", at)
                _float(mixer, "tau", at)
            else:
                _int(mixer, "inner", at), _int(mixer, "state", at), _int(mixer, "dt_rank", at), _int(mixer, "conv", at)
            mlp = layer.get("mlp")
            if mlp is not None:
                at = where + "mlp."
                if mlp.get("kind") != "moe":
                    raise ConfigError(f"config.json: {at}kind must be 'moe', got {mlp.get('kind')!r}")
                expert = _section(mlp, "expert", at)
                _int(expert, "ff", at + "expert.")
                _float(expert, "limit", at + "expert.")
                router = _section(mlp, "router", at)
                experts, top = _int(router, "experts", at + "router."), _int(router, "top", at + "router.")
                if top > experts:
                    raise ConfigError(f"config.json: {at}router.top {top} is more than the {experts} experts")
                if mlp.get("shared") is not None:
                    _int(mlp["shared"], "ff", at + "shared.")
                    _float(mlp["shared"], "limit", at + "shared.")

    def to_dict(self) -> dict:
        def thaw(value):
            if isinstance(value, Mapping):
                return {k: thaw(v) for k, v in value.items()}
            if isinstance(value, tuple):
                return [thaw(v) for v in value]
            return value
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps},
               "layers": [thaw(layer) for layer in self.layers]}
        if self.streams is not None:
            out["streams"] = self.streams
        return out

    # ------------------------------------------------------------------ the plan

    def _norm(self, name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"size": self.width, "eps": self.norm_eps, "residual": "float32", "gain": "scalar"},
                        {"weight": name})

    def _mixer(self, layer: Mapping[str, Any], prefix: str) -> PartSpec:
        m, kind = layer["mixer"], layer["type"]
        if kind == MAMBA:
            t = {key: f"{prefix}mix.{name}" for key, name in (
                ("in", "in"), ("conv", "conv"), ("conv_bias", "conv.b"), ("x", "x"), ("dt", "dt"), ("dt_bias", "dt.b"),
                ("A_log", "A_log"), ("D", "D"), ("o", "o"))}
            return PartSpec("selective_scan", {"hidden_size": self.width, "inner": m["inner"], "state": m["state"],
                                               "dt_rank": m["dt_rank"], "conv_taps": m["conv"]}, t)
        if kind == GLA:
            t = {key: f"{prefix}mix.{name}" for key, name in (
                ("q", "q"), ("k", "k"), ("v", "v"), ("g", "g"), ("o", "o"), ("norm", "norm"), ("a1", "a1"), ("a2", "a2"),
                ("a2_bias", "a2.b"))}
            return PartSpec("linear_attention",
                            {"hidden_size": self.width, "n_heads": m["heads"], "key_dim": m["dim"], "value_dim": m["vdim"],
                             "decay": {"kind": "gated", "rank": m.get("rank"), "tau": float(m["tau"])},
                             "q_scale": float(m["dim"]) ** -0.5, "silu_inputs": False, "norm_scope": "head",
                             "norm_eps": self.norm_eps, "gate": "silu"}, t)
        left, right = m["left"], m["right"]
        rot = left["rot"]
        position = None
        if rot["dims"]:
            position = PartSpec("rope", {"head_dim": left["dim"], "rotary_dim": rot["dims"], "theta": float(rot["base"]),
                                         "layout": "half", "frequency_precision": "float64",
                                         "angle_precision": "float64"})
        value_position = PartSpec("rope", {"head_dim": left["vdim"], "rotary_dim": left["vdim"], "theta": float(rot["base"]),
                                           "layout": "half", "frequency_precision": "float64",
                                           "angle_precision": "float64"})
        lt = {key: f"{prefix}mix.left.{name}" for key, name in (
            ("q_proj", "q"), ("k_proj", "k"), ("v_proj", "v"), ("o_proj", "o"), ("q_bias", "q.b"), ("k_bias", "k.b"),
            ("v_bias", "v.b"), ("o_bias", "o.b"), ("sink", "sink"), ("g_proj", "g"))}
        rt = {key: f"{prefix}mix.right.{name}" for key, name in (
            ("q", "q"), ("k", "k"), ("v", "v"), ("g", "g"), ("o", "o"), ("norm", "norm"))}
        return PartSpec("mixer_pair", {
            "left": PartSpec("gated_attention",
                             {"hidden_size": self.width, "n_heads": left["heads"], "n_kv_heads": left["kv_heads"],
                              "head_dim": left["dim"], "value_dim": left["vdim"], "scale": float(left["scale"]),
                              "qk_norm_eps": self.norm_eps, "position": position, "value_position": value_position,
                              "biases": True, "sinks": True, "gate": "logistic"}, lt),
            "right": PartSpec("linear_attention",
                              {"hidden_size": self.width, "n_heads": right["heads"], "key_dim": right["dim"],
                               "value_dim": right["vdim"],
                               "decay": {"kind": "constant", "values": [float(v) for v in right["decay"]]},
                               "q_scale": 1.0, "silu_inputs": True, "norm_scope": "all", "norm_eps": self.norm_eps,
                               "gate": "logistic"}, rt),
            "left_scale": float(m["left_scale"]), "right_scale": float(m["right_scale"])})

    def _ffn(self, mlp: Mapping[str, Any], prefix: str) -> PartSpec:
        router, shared = mlp["router"], mlp.get("shared")
        tensors = {"router": prefix + "mlp.router"}
        for e in range(router["experts"]):
            tensors[f"gate.{e}"] = f"{prefix}mlp.e{e}.gate"
            tensors[f"up.{e}"] = f"{prefix}mlp.e{e}.up"
            tensors[f"down.{e}"] = f"{prefix}mlp.e{e}.down"
        if shared is not None:
            tensors.update(shared_gate_proj=prefix + "mlp.shared.gate", shared_up=prefix + "mlp.shared.up",
                           shared_down=prefix + "mlp.shared.down")
        return PartSpec(
            "routed_clamped_experts",
            {"hidden_size": self.width, "n_experts": router["experts"], "expert_ff": mlp["expert"]["ff"],
             "top": router["top"], "limit": float(mlp["expert"]["limit"]), "slope": EXPERT_GATE_SLOPE,
             "shared_ff": 0 if shared is None else shared["ff"],
             "shared_limit": None if shared is None else float(shared["limit"]), "shared_gated": False,
             "scoring": "softmax", "renormalise": ROUTER_SUM_FLOOR, "weight_at": "output"},
            tensors)

    def plan(self) -> ModelPlan:
        layers: List[LayerSpec] = []
        schedule: List[ScheduleEntry] = []
        connected = self.streams is not None
        for i, layer in enumerate(self.layers):
            prefix = f"l{i}."
            parts = dict(mixer=self._mixer(layer, prefix), norm_mixer=self._norm(prefix + "norm1"))
            tensors = {}
            if connected:
                tensors.update({"mixer.read": prefix + "hc1.in", "mixer.mix": prefix + "hc1.mix",
                                "mixer.write": prefix + "hc1.out"})
            if layer.get("mlp") is not None:
                parts.update(ffn=self._ffn(layer["mlp"], prefix), norm_ffn=self._norm(prefix + "norm2"))
                if connected:
                    tensors.update({"ffn.read": prefix + "hc2.in", "ffn.mix": prefix + "hc2.mix",
                                    "ffn.write": prefix + "hc2.out"})
            block = PartSpec("hyper_connections", dict(parts, streams=self.streams or 1, connections=connected), tensors)
            layers.append(LayerSpec(block))
            schedule.append(ScheduleEntry(layer=i, cache=i))
        return ModelPlan(
            hidden_size=self.width,
            vocab_size=self.vocab,
            embedding=PartSpec("embedding", {"vocab_size": self.vocab, "hidden_size": self.width,
                                             "scale": self.embedding_scale, "stream": "float32"}, {"weight": "embed"}),
            layers=tuple(layers),
            schedule=tuple(schedule),
            final_norm=self._norm("final.norm"),
            head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": self.width, "tied": False},
                          {"weight": "head"}),
            max_positions=self.max_positions,
        )
