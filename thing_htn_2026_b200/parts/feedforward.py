"""Dense feed-forward with a gated SiLU: ``down(silu(gate(x)) * up(x))``.  Gate and up
are one product over the concatenated weight ``[2I, H]`` (engine/engine.py:221, :1116-1118);
the activation rounds as engine/kernels/torch_ref.py:74-88 does.

``clamped_glu``: ``down(g * logistic(slope * g) * (u + 1))`` with ``g = min(gate(x), limit)`` and
``u = clamp(up(x), -limit, limit)``; ``limit`` and ``slope`` are parameters.

``routed_experts``: a mixture of ``n_experts`` experts ``down_e(gelu(up_e(x)))`` (the exact gelu,
no biases) of which a token uses ``top``.  Router logits ``z = router(x)`` and scores
``s = softmax(z)`` over all experts are float32; the experts form ``groups`` equal groups of
neighbours, a group's score is its largest ``s``, only experts of the ``keep`` best groups can be
chosen, and the chosen are the ``top`` allowed experts with the largest ``s``; a chosen expert's
output is weighted by ``s * scale`` (not renormalised).  With ``shared_ff`` a shared expert of
the same form runs for every token and is added, multiplied by ``logistic(shared_gate(x))`` (one
number per token; ``shared_gated`` False: added as it is).  The up-projections of all experts are
one product, the activation carries the routing weights (zero for an expert that was not chosen),
and one down-projection over all experts' columns sums the chosen ones: the result does not
depend on the other rows of the step.  Kernels: csrc/moe.cu.

``polynorm``: ``down(act(up(x)))`` with ``act(z) = a N(z) + b N(z^2) + c N(z^3) + e``, powers
taken entry by entry and ``N`` the division of a token's vector by its root mean square (``eps``
inside the root); the four numbers are a tensor of the layer (``act``).

``routed_clamped_experts``: a mixture whose experts have the form of ``clamped_glu`` (``limit``,
``slope``).  Scores are ``logistic(router(x))``, each expert by itself, in float32; the ``top``
largest are chosen and weighted by their scores as they are.  The weight multiplies the expert's
*input*: the output is the sum of ``expert(w x)``.  Because the projections are linear, the gate
and up projections of all experts are one product over ``x`` and the activation kernel multiplies
the projected values by ``w`` before the clamps; one down-projection over all experts' columns
sums the chosen ones.  With ``shared_ff`` a shared expert with a limit of its own
(``shared_limit``) runs for every token on the token itself and is added times
``logistic(shared_gate(x))`` (``shared_gated`` False: added as it is).  ``scoring`` "softmax": the
scores are a softmax over all experts instead; ``renormalise`` (a small number): the chosen
experts' scores are divided by their sum plus that number; ``weight_at`` "output": an expert sees
the token itself and its output is weighted (the weight then multiplies the activation, ahead of
the one down-projection over all columns)."""

from __future__ import annotations

from typing import List

import torch

from .. import ops
from ..config.base import PartSpec
from ..weights.loader import GAIN, MATRIX, TensorSpec
from .registry import register_part
from .runtime import Runtime


@register_part("ffn", "swiglu")
class SwiGLU:
    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> List[TensorSpec]:
        hidden, inter = int(spec.params["hidden_size"]), int(spec.params["intermediate_size"])
        return [TensorSpec(spec.tensors["gate_proj"], (inter, hidden), MATRIX),
                TensorSpec(spec.tensors["up_proj"], (inter, hidden), MATRIX),
                TensorSpec(spec.tensors["down_proj"], (hidden, inter), MATRIX)]

    def __init__(self, spec: PartSpec, runtime: Runtime):
        self.w_gate_up = torch.cat([runtime.tensor(spec, "gate_proj"), runtime.tensor(spec, "up_proj")], dim=0).contiguous()
        self.w_down = runtime.tensor(spec, "down_proj")

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        err = getattr(ctx, "err", None)
        return ops.linear(ops.linear_swiglu(x, self.w_gate_up, err), self.w_down, err=err)


@register_part("ffn", "clamped_glu")
class ClampedGLU:
    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> List[TensorSpec]:
        return SwiGLU.tensor_specs(spec)

    def __init__(self, spec: PartSpec, runtime: Runtime):
        self.limit, self.slope = float(spec.params["limit"]), float(spec.params["slope"])
        self.w_gate_up = torch.cat([runtime.tensor(spec, "gate_proj"), runtime.tensor(spec, "up_proj")], dim=0).contiguous()
        self.w_down = runtime.tensor(spec, "down_proj")

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        err = getattr(ctx, "err", None)
        y = ops.clamped_glu(ops.linear(x, self.w_gate_up, err=err), self.limit, self.slope)
        return ops.linear(y, self.w_down, err=err)


@register_part("ffn", "routed_experts")
class RoutedExperts:
    @staticmethod
    def _sizes(spec: PartSpec):
        p = spec.params
        return int(p["hidden_size"]), int(p["n_experts"]), int(p["expert_ff"]), int(p.get("shared_ff") or 0)

    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> List[TensorSpec]:
        hidden, n, ff, shared = cls._sizes(spec)
        specs = [TensorSpec(spec.tensors["router"], (n, hidden), MATRIX)]
        for e in range(n):
            specs += [TensorSpec(spec.tensors[f"up.{e}"], (ff, hidden), MATRIX),
                      TensorSpec(spec.tensors[f"down.{e}"], (hidden, ff), MATRIX)]
        if shared:
            specs += [TensorSpec(spec.tensors["shared_up"], (shared, hidden), MATRIX),
                      TensorSpec(spec.tensors["shared_down"], (hidden, shared), MATRIX)]
            if spec.params.get("shared_gated", True):
                specs.append(TensorSpec(spec.tensors["shared_gate"], (1, hidden), MATRIX))
        return specs

    def __init__(self, spec: PartSpec, runtime: Runtime):
        p = spec.params
        _, self.n_experts, self.ff, self.shared_ff = self._sizes(spec)
        self.top, self.scale = int(p["top"]), float(p.get("scale", 1.0))
        self.groups, self.keep = int(p.get("groups") or 1), int(p.get("keep") or p.get("groups") or 1)
        if self.n_experts % self.groups or not 0 < self.keep <= self.groups \
                or not 0 < self.top <= self.keep * (self.n_experts // self.groups):
            raise ValueError(f"routed_experts: top {self.top} of {self.n_experts} experts in {self.groups} groups, "
                             f"{self.keep} kept")
        self.shared_gated = bool(self.shared_ff) and bool(p.get("shared_gated", True))
        ups = [runtime.tensor(spec, f"up.{e}") for e in range(self.n_experts)]
        downs = [runtime.tensor(spec, f"down.{e}") for e in range(self.n_experts)]
        route = [runtime.tensor(spec, "router")]
        if self.shared_ff:
            ups.append(runtime.tensor(spec, "shared_up"))
            downs.append(runtime.tensor(spec, "shared_down"))
        if self.shared_gated:
            route.append(runtime.tensor(spec, "shared_gate"))
        self.w_up = torch.cat(ups, dim=0).contiguous()
        self.w_down = torch.cat(downs, dim=1).contiguous()
        self.w_route = torch.cat(route, dim=0).contiguous()

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        err = getattr(ctx, "err", None)
        z = ops.linear(x, self.w_route, out_dtype=torch.float32, err=err)
        routing = ops.moe_route(z, self.n_experts, self.groups, self.keep, self.top, self.scale)
        u = ops.linear(x, self.w_up, err=err)
        a = ops.routed_gelu(u, routing, self.ff, self.shared_ff, z if self.shared_gated else None, self.n_experts)
        return ops.linear(a, self.w_down, err=err)


@register_part("ffn", "polynorm")
class PolyNormFFN:
    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> List[TensorSpec]:
        hidden, inter = int(spec.params["hidden_size"]), int(spec.params["intermediate_size"])
        return [TensorSpec(spec.tensors["up_proj"], (inter, hidden), MATRIX),
                TensorSpec(spec.tensors["down_proj"], (hidden, inter), MATRIX),
                TensorSpec(spec.tensors["act"], (4,), GAIN, init="polynomial")]

    def __init__(self, spec: PartSpec, runtime: Runtime):
        self.eps = float(spec.params["eps"])
        self.w_up = runtime.tensor(spec, "up_proj")
        self.w_down = runtime.tensor(spec, "down_proj")
        self.coefficients = runtime.tensor(spec, "act").to(torch.float32).contiguous()

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        err = getattr(ctx, "err", None)
        return ops.linear(ops.polynorm(ops.linear(x, self.w_up, err=err), self.coefficients, self.eps), self.w_down, err=err)


@register_part("ffn", "routed_clamped_experts")
class RoutedClampedExperts:
    @staticmethod
    def _sizes(spec: PartSpec):
        p = spec.params
        return int(p["hidden_size"]), int(p["n_experts"]), int(p["expert_ff"]), int(p.get("shared_ff") or 0)

    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> List[TensorSpec]:
        hidden, n, ff, shared = cls._sizes(spec)
        specs = [TensorSpec(spec.tensors["router"], (n, hidden), MATRIX)]
        for e in range(n):
            specs += [TensorSpec(spec.tensors[f"gate.{e}"], (ff, hidden), MATRIX),
                      TensorSpec(spec.tensors[f"up.{e}"], (ff, hidden), MATRIX),
                      TensorSpec(spec.tensors[f"down.{e}"], (hidden, ff), MATRIX)]
        if shared:
            specs += [TensorSpec(spec.tensors["shared_gate_proj"], (shared, hidden), MATRIX),
                      TensorSpec(spec.tensors["shared_up"], (shared, hidden), MATRIX),
                      TensorSpec(spec.tensors["shared_down"], (hidden, shared), MATRIX)]
            if spec.params.get("shared_gated", True):
                specs.append(TensorSpec(spec.tensors["shared_gate"], (1, hidden), MATRIX))
        return specs

    def __init__(self, spec: PartSpec, runtime: Runtime):
        p = spec.params
        _, self.n_experts, self.ff, self.shared_ff = self._sizes(spec)
        self.top = int(p["top"])
        if not 0 < self.top <= self.n_experts:
            raise ValueError(f"routed_clamped_experts: top {self.top} of {self.n_experts} experts")
        self.limit, self.slope = float(p["limit"]), float(p["slope"])
        self.shared_limit = float(p.get("shared_limit") or self.limit)
        self.scoring = str(p.get("scoring", "logistic"))
        self.renormalise = None if p.get("renormalise") is None else float(p["renormalise"])
        self.weight_at = str(p.get("weight_at", "input"))
        if self.scoring not in ops.SCORINGS or self.weight_at not in ("input", "output") \
                or (self.renormalise is not None and self.scoring != "softmax"):
            raise ValueError(f"routed_clamped_experts: scoring {self.scoring!r}, weight_at {self.weight_at!r}, "
                             f"renormalise {self.renormalise!r}")
        self.shared_gated = bool(self.shared_ff) and bool(p.get("shared_gated", True))
        gates = [runtime.tensor(spec, f"gate.{e}") for e in range(self.n_experts)]
        ups = [runtime.tensor(spec, f"up.{e}") for e in range(self.n_experts)]
        downs = [runtime.tensor(spec, f"down.{e}") for e in range(self.n_experts)]
        route = [runtime.tensor(spec, "router")]
        if self.shared_ff:
            gates.append(runtime.tensor(spec, "shared_gate_proj"))
            ups.append(runtime.tensor(spec, "shared_up"))
            downs.append(runtime.tensor(spec, "shared_down"))
        if self.shared_gated:
            route.append(runtime.tensor(spec, "shared_gate"))
        self.w_gate_up = torch.cat(gates + ups, dim=0).contiguous()     # the gates of all columns, then the ups
        self.w_down = torch.cat(downs, dim=1).contiguous()
        self.w_route = torch.cat(route, dim=0).contiguous()

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        err = getattr(ctx, "err", None)
        z = ops.linear(x, self.w_route, out_dtype=torch.float32, err=err)
        routing = ops.moe_route(z, self.n_experts, 1, 1, self.top, 1.0, scoring=self.scoring, renormalise=self.renormalise)
        gu = ops.linear(x, self.w_gate_up, err=err)
        y = ops.routed_clamped_glu(gu, routing, self.ff, self.shared_ff, self.limit, self.shared_limit, self.slope,
                                   z if self.shared_gated else None, self.n_experts, weight_at=self.weight_at)
        return ops.linear(y, self.w_down, err=err)
