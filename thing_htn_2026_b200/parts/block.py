"""Arrangement of a layer's parts.  ``pre_norm``: ``a = x + mixer(norm(x))``,
``y = a + ffn(norm(a))`` (OPTIMIZATION_GUIDE.md:57-70).  The add of a branch's output is
deferred to the next norm, which fuses it (engine/engine.py:1104-1118): a block takes and
returns the pair (residual stream ``h``, pending branch output ``d`` or None).

A block owns its sub-parts.  Their specs are parameters of the block's own spec, the block
builds them, lists their tensors, answers for their cache need and passes on what they
ask of a step.  The model above sees blocks only, so an arrangement with other members is
a new class of this family and nothing else.

``sandwich_norm``: a norm on both sides of every sublayer, ``a = x + post(mixer(norm(x)))``,
``y = a + post'(ffn(norm'(a)))``, over a residual stream kept in float32; the feed-forward
half may be absent.  The pending output travels as a :class:`Branch` that names the norm it
still has to pass, so that this norm, the add and the next norm are one kernel.

``branch_norm``: the norm stands on a sublayer's output only and the sublayers read the stream
itself: ``a = x + norm(mixer(x))``, ``y = a + norm'(ffn(a))``, over a float32 stream; the
feed-forward half may be absent.  The pending output again travels as a :class:`Branch`, and
"norm of the branch, add, round the sum for the next sublayer" is one kernel.

``parallel``: one norm per layer, read by both sublayers: ``n = norm(x)``,
``y = x + factor * (mixer(n) + ffn(n))`` over a float32 stream (``factor`` a parameter of the
block, default 1; the feed-forward may be absent).  The two outputs travel as one
:class:`Branch` with its second tensor and its factor, so that "add both, times the factor, into
the stream, norm of the sum" is one kernel at the next layer's norm or at the model's last.

``hyper_connections``: the residual stream is ``streams`` copies ``X_0 .. X_(s-1)`` in float32,
all equal to the embedding's row at the start.  A sublayer f with the numbers ``read[s]``,
``mix[s, s]`` ([from, to]) and ``write[s]`` does ``u = sum_j read[j] X_j``, ``y = f(norm(u))``,
``X'_i = sum_j mix[j, i] X_j + write[i] y``; a layer is its mixer as such a sublayer, then its
feed-forward where it has one.  The pending output travels as a :class:`Branch` with the numbers
of its write, so that "write of the last sublayer, read of the next, its norm" is one kernel
(:func:`ops.hyper_norm`), also into the model's last norm, which reads the sum of the copies.
Without the numbers' tensors (``connections`` False) it is one copy and the plain
``x <- x + f(norm(x))``.
"""

from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..cache.sequence_cache import CacheNeed
from ..config.base import PartSpec, ScheduleEntry
from .. import ops
from ..weights.loader import GAIN, TensorSpec
from .registry import part_class, register_part
from .runtime import Branch, HostBatch, Runtime, StepContext


class Block:
    """Base of the block arrangements.  ``MEMBERS`` maps the names of the sub-part specs among
    the block's parameters to their families; a member whose spec is absent or None is left
    out (the attribute of that name is None)."""

    MEMBERS: Dict[str, str] = {}

    @classmethod
    def members(cls, spec: PartSpec) -> List[Tuple[str, str, PartSpec]]:
        return [(name, family, spec.params[name]) for name, family in cls.MEMBERS.items()
                if spec.params.get(name) is not None]

    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> List[TensorSpec]:
        specs: List[TensorSpec] = []
        for _, family, member in cls.members(spec):
            specs += part_class(family, member.kind).tensor_specs(member)
        return specs

    def __init__(self, spec: PartSpec, runtime: Runtime):
        for name in self.MEMBERS:
            setattr(self, name, None)
        for name, family, member in self.members(spec):
            setattr(self, name, part_class(family, member.kind)(member, runtime))

    def parts(self) -> List[object]:
        return [getattr(self, name) for name in self.MEMBERS if getattr(self, name) is not None]

    def cache_need(self) -> CacheNeed:
        """What the block's cache entry stores: the need of its (one) mixer."""
        mixer = getattr(self, "mixer", None)
        return mixer.cache_need() if mixer is not None else None

    def step_inputs(self, batch: HostBatch, out: Dict[str, List[int]]) -> None:
        """Integer inputs that members want computed on the host for this step, by name."""
        for part in self.parts():
            if hasattr(part, "step_inputs"):
                part.step_inputs(batch, out)


@register_part("block", "pre_norm")
class PreNormBlock(Block):
    MEMBERS = {"norm_mixer": "norm", "mixer": "mixer", "norm_ffn": "norm", "ffn": "ffn"}

    def forward(self, h: torch.Tensor, d: Optional[torch.Tensor], ctx: StepContext,
                entry: ScheduleEntry) -> Tuple[torch.Tensor, torch.Tensor]:
        n = self.norm_mixer.forward(h) if d is None else self.norm_mixer.add_forward(h, d)
        a = self.mixer.forward(n, ctx, entry)
        n = self.norm_ffn.add_forward(h, a)
        return h, self.ffn.forward(n, ctx)


@register_part("block", "sandwich_norm")
class SandwichNormBlock(Block):
    MEMBERS = {"norm_mixer": "norm", "mixer": "mixer", "post_norm_mixer": "norm",
               "norm_ffn": "norm", "ffn": "ffn", "post_norm_ffn": "norm"}

    def forward(self, h: torch.Tensor, d, ctx: StepContext, entry: ScheduleEntry):
        if d is None:
            if h.dtype == torch.float32:
                n = self.norm_mixer.forward(h)
            else:                      # the embedding's rows start the float32 stream
                h, n = self.norm_mixer.start_forward(h)
        elif isinstance(d, Branch):
            n = self.norm_mixer.add_forward(h, d.tensor, post=d.norm)
        else:
            n = self.norm_mixer.add_forward(h, d)
        a = Branch(self.mixer.forward(n, ctx, entry), self.post_norm_mixer)
        if self.ffn is None:
            return h, a
        n = self.norm_ffn.add_forward(h, a.tensor, post=a.norm)
        return h, Branch(self.ffn.forward(n, ctx), self.post_norm_ffn)


@register_part("block", "branch_norm")
class BranchNormBlock(Block):
    MEMBERS = {"mixer": "mixer", "norm_mixer": "norm", "ffn": "ffn", "norm_ffn": "norm"}

    def forward(self, h: torch.Tensor, d, ctx: StepContext, entry: ScheduleEntry):
        if h.dtype != torch.float32:
            raise TypeError("branch_norm: the residual stream must start in float32 (an embedding with stream 'float32')")
        if d is None:
            x = self.norm_mixer.read(h)
        elif isinstance(d, Branch) and d.norm is not None:
            x = d.norm.add_read(h, d.tensor)
        else:
            raise TypeError("branch_norm: a pending branch must name the norm it passes before the add")
        a = Branch(self.mixer.forward(x, ctx, entry), self.norm_mixer)
        if self.ffn is None:
            return h, a
        x = self.norm_mixer.add_read(h, a.tensor)
        return h, Branch(self.ffn.forward(x, ctx), self.norm_ffn)


@register_part("block", "parallel")
class ParallelBlock(Block):
    MEMBERS = {"norm": "norm", "mixer": "mixer", "ffn": "ffn"}

    def __init__(self, spec: PartSpec, runtime: Runtime):
        super().__init__(spec, runtime)
        self.factor = float(spec.params.get("factor", 1.0))

    def forward(self, h: torch.Tensor, d, ctx: StepContext, entry: ScheduleEntry):
        if h.dtype != torch.float32:
            raise TypeError("parallel: the residual stream must start in float32 (an embedding with stream 'float32')")
        if d is None:
            n = self.norm.forward(h)
        elif isinstance(d, Branch):
            n = self.norm.add_forward(h, d, post=d.norm)
        else:
            n = self.norm.add_forward(h, d)
        a = self.mixer.forward(n, ctx, entry)
        f = self.ffn.forward(n, ctx) if self.ffn is not None else None
        return h, Branch(a, None, f, self.factor)


@register_part("block", "hyper_connections")
class HyperConnectionBlock(Block):
    MEMBERS = {"norm_mixer": "norm", "mixer": "mixer", "norm_ffn": "norm", "ffn": "ffn"}
    SUBLAYERS = ("mixer", "ffn")

    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> List[TensorSpec]:
        specs = super().tensor_specs(spec)
        s = int(spec.params.get("streams") or 1)
        if spec.params.get("connections", True):
            for name in cls.SUBLAYERS:
                if spec.params.get(name) is None:
                    continue
                specs += [TensorSpec(spec.tensors[f"{name}.read"], (s,), GAIN, init="stream_read"),
                          TensorSpec(spec.tensors[f"{name}.write"], (s,), GAIN),
                          TensorSpec(spec.tensors[f"{name}.mix"], (s, s), GAIN, init="stream_mix")]
        return specs

    def __init__(self, spec: PartSpec, runtime: Runtime):
        super().__init__(spec, runtime)
        self.streams = s = int(spec.params.get("streams") or 1)
        self.numbers = {}
        f32 = lambda t: t.to(torch.float32).contiguous()
        for name in self.SUBLAYERS:
            if spec.params.get(name) is None:
                continue
            if spec.params.get("connections", True):
                self.numbers[name] = ops.StreamNumbers(f32(runtime.tensor(spec, f"{name}.read")),
                                                       f32(runtime.tensor(spec, f"{name}.mix")),
                                                       f32(runtime.tensor(spec, f"{name}.write")))
            else:
                if s != 1:
                    raise ValueError("hyper_connections: several streams need the numbers that connect them")
                one = torch.ones(1, dtype=torch.float32, device=runtime.device)
                self.numbers[name] = ops.StreamNumbers(one, one.reshape(1, 1), one)

    def forward(self, h: torch.Tensor, d, ctx: StepContext, entry: ScheduleEntry):
        if h.dtype != torch.float32:
            raise TypeError("hyper_connections: the residual stream must start in float32 (an embedding with stream 'float32')")
        own = self.numbers["mixer"]
        if d is None:           # the model's first layer: every copy starts as the embedding's row
            X, n = self.norm_mixer.stream_norm(None, self.streams, start=h, read=own.read)
        elif isinstance(d, Branch) and d.write is not None:
            X, n = self.norm_mixer.stream_norm(h, self.streams, y=d.tensor, written=d.write, read=own.read)
        else:
            raise TypeError("hyper_connections: a pending branch must carry the numbers of its write")
        a = self.mixer.forward(n, ctx, entry)
        if self.ffn is None:
            return X, Branch(a, write=own)
        after = self.numbers["ffn"]
        X, n = self.norm_ffn.stream_norm(X, self.streams, y=a, written=own, read=after.read)
        return X, Branch(self.ffn.forward(n, ctx), write=after)
