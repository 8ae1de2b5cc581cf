"""Mixers in three phases, so that several can share their products.

A mixer of this kind says which rows of an input projection it wants (``in_rows``: a weight
``[n, hidden]`` and an optional bias), turns its columns of the projected rows into the
activation that its output projection reads (``inner``: written, times a constant, into columns of
a buffer that may be shared), and says what projects that back (``out_rows``: a weight
``[hidden, inner_width]`` and an optional bias).  Alone, :class:`PhasedMixer.forward` runs the three
phases with products of its own.  ``mixer_pair`` runs two such mixers side by side on the same
input, ``y = left_scale * left(x) + right_scale * right(x)``: ONE input product over both mixers'
rows, their activations side by side in one buffer with the scales applied there (float32, before
the one rounding), and ONE output product over the concatenated columns, whose bias is the scaled
sum of theirs.  The pair's cache entry holds what both need (keys and values of the one, state
tensors of the other).
"""

from __future__ import annotations

from typing import List, Optional, Tuple

import torch

from .. import ops
from ..cache.sequence_cache import CacheNeed, KVSpec
from ..config.base import PartSpec, ScheduleEntry
from ..weights.loader import TensorSpec
from .registry import part_class, register_part
from .runtime import Runtime, StepContext


def cat_bias(pieces: List[Tuple[torch.Tensor, Optional[torch.Tensor]]]) -> Optional[torch.Tensor]:
    """The biases of weights stacked along their rows, zeros where a weight has none; None if none has."""
    if all(b is None for _, b in pieces):
        return None
    return torch.cat([b if b is not None else torch.zeros(w.shape[0], dtype=w.dtype, device=w.device)
                      for w, b in pieces]).contiguous()


class PhasedMixer:
    """Base of the mixers in three phases.  ``state_base``: the index of this mixer's first state
    tensor in its cache entry (a pair moves the second mixer's behind the first's)."""

    inner_width: int = 0
    state_base: int = 0

    def in_rows(self) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        raise NotImplementedError

    def out_rows(self) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        raise NotImplementedError

    def inner(self, x: torch.Tensor, proj: torch.Tensor, offset: int, ctx: StepContext, entry: ScheduleEntry,
              out: torch.Tensor, out_offset: int, scale: float) -> None:
        raise NotImplementedError

    def finish(self) -> None:
        """Called once the weights are where they will be used: alone, this mixer's own products."""
        self.w_in, self.b_in = self.in_rows()
        self.w_out, self.b_out = self.out_rows()

    def forward(self, x: torch.Tensor, ctx: StepContext, entry: ScheduleEntry) -> torch.Tensor:
        proj = ops.linear(x, self.w_in, err=ctx.err, bias=self.b_in)
        z = torch.empty((x.shape[0], self.inner_width), dtype=x.dtype, device=x.device)
        self.inner(x, proj, 0, ctx, entry, z, 0, 1.0)
        return ops.linear(z, self.w_out, err=ctx.err, bias=self.b_out)


@register_part("mixer", "mixer_pair")
class MixerPair:
    MEMBERS = ("left", "right")

    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> List[TensorSpec]:
        specs: List[TensorSpec] = []
        for name in cls.MEMBERS:
            member = spec.params[name]
            specs += part_class("mixer", member.kind).tensor_specs(member)
        return specs

    def __init__(self, spec: PartSpec, runtime: Runtime):
        self.members = [part_class("mixer", spec.params[name].kind)(spec.params[name], runtime) for name in self.MEMBERS]
        for member in self.members:
            if not isinstance(member, PhasedMixer):
                raise TypeError("mixer_pair: both mixers must work in phases (in_rows, inner, out_rows)")
        self.scales = [float(spec.params.get(name + "_scale", 1.0)) for name in self.MEMBERS]
        ins = [m.in_rows() for m in self.members]
        outs = [m.out_rows() for m in self.members]
        self.w_in = torch.cat([w for w, _ in ins], dim=0).contiguous()
        self.b_in = cat_bias(ins)
        self.w_out = torch.cat([w for w, _ in outs], dim=1).contiguous()
        self.b_out = None
        if any(b is not None for _, b in outs):
            total = sum(b.to(torch.float32) * scale for (_, b), scale in zip(outs, self.scales) if b is not None)
            self.b_out = total.to(self.w_out.dtype).contiguous()
        self.in_offsets, self.out_offsets, at_in, at_out, states = [], [], 0, 0, 0
        for member, (w, _) in zip(self.members, ins):
            self.in_offsets.append(at_in)
            self.out_offsets.append(at_out)
            at_in += w.shape[0]
            at_out += member.inner_width
            member.state_base = states
            need = member.cache_need()
            states += sum(not isinstance(one, KVSpec) for one in (need if isinstance(need, tuple) else (need,))
                          if one is not None)
        self.inner_width = at_out

    def cache_need(self) -> CacheNeed:
        needs = []
        for member in self.members:
            need = member.cache_need()
            needs += [one for one in (need if isinstance(need, tuple) else (need,)) if one is not None]
        return tuple(needs) if needs else None

    def step_inputs(self, batch, out) -> None:
        for member in self.members:
            if hasattr(member, "step_inputs"):
                member.step_inputs(batch, out)

    def forward(self, x: torch.Tensor, ctx: StepContext, entry: ScheduleEntry) -> torch.Tensor:
        proj = ops.linear(x, self.w_in, err=ctx.err, bias=self.b_in)
        z = torch.empty((x.shape[0], self.inner_width), dtype=x.dtype, device=x.device)
        for member, at_in, at_out, scale in zip(self.members, self.in_offsets, self.out_offsets, self.scales):
            member.inner(x, proj, at_in, ctx, entry, z, at_out, scale)
        return ops.linear(z, self.w_out, err=ctx.err, bias=self.b_out)
