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
"""

from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..cache.sequence_cache import CacheNeed
from ..config.base import PartSpec, ScheduleEntry
from ..weights.loader import TensorSpec
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
