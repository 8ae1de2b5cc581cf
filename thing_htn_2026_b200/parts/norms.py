"""RMSNorm.  ``forward`` normalises; ``add_forward`` first adds a branch's output to the
residual stream in place (the reference fuses the two the same way,
engine/kernels/torch_ref.py:61-68, engine/engine.py:1104-1107).

Parameters: ``size``, ``eps``; ``gain_offset`` (default 0; 1 for a gain stored around zero,
which multiplies as ``1 + w``); ``residual`` (default: the activation type; "float32": the
stream this norm reads is kept in float32 whatever the activation type, and every sum of the
norm is float32 with one rounding at the output).  With a float32 stream, ``add_forward``
also takes ``post``: another norm of this kind that the branch's output passes before it is
added (norms on both sides of a sublayer), in the same kernel.  ``groups`` (default 1; float32
stream only): the row is split into that many equal consecutive parts, each divided by its own
``sqrt(mean(part^2) + eps)``, and the whole is multiplied by the gain.  ``add_forward`` takes a
:class:`Branch` as well: its second tensor and its factor are added in the same kernel,
``h <- h + factor * (d + d')``.  ``gain`` "scalar": the gain is one number (a tensor without
axes) for all coordinates.  ``stream_norm`` serves a residual stream of several copies
(hyper-connections, :func:`ops.hyper_norm`): the pending write of the sublayer before, the read of
the next one and this norm of what was read, in one kernel.

``layernorm``: ``(x - mean) / sqrt(var + eps) * w + b`` with the variance as the mean of the
squared deviations, over a float32 stream only.  Besides the calls above it has ``read`` and
``add_read`` for arrangements whose sublayers read the stream itself, with the norm on a
sublayer's output: ``add_read(h, d)`` does ``h <- h + self(d)`` and returns ``h`` rounded to the
activation type, in one kernel."""

from __future__ import annotations

from typing import List, Optional

import torch

from .. import ops
from ..config.base import PartSpec
from ..weights.loader import GAIN, TensorSpec
from .registry import register_part
from .runtime import Branch, Runtime


@register_part("norm", "rmsnorm")
class RMSNorm:
    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> List[TensorSpec]:
        init = "zero_centered" if float(spec.params.get("gain_offset", 0.0)) else None
        shape = () if spec.params.get("gain") == "scalar" else (int(spec.params["size"]),)
        return [TensorSpec(spec.tensors["weight"], shape, GAIN, init=init)]

    def __init__(self, spec: PartSpec, runtime: Runtime):
        self.size = int(spec.params["size"])
        self.eps = float(spec.params["eps"])
        self.offset = float(spec.params.get("gain_offset", 0.0))
        self.float32_stream = spec.params.get("residual") == "float32"
        self.groups = int(spec.params.get("groups") or 1)
        if self.groups < 1 or self.size % self.groups or (self.groups > 1 and not self.float32_stream):
            raise ValueError(f"rmsnorm: {self.groups} groups must divide the size {self.size} and need a float32 stream")
        self.dtype = runtime.dtype
        self.gain = runtime.tensor(spec, "weight")
        self.scalar_gain = spec.params.get("gain") == "scalar"
        if self.scalar_gain:
            if not self.float32_stream or self.offset or self.groups != 1:
                raise ValueError("rmsnorm: a gain of one number goes with a float32 stream, no offset and no groups")
            self.gain32 = self.gain.to(torch.float32).reshape(1).contiguous()
            self._ones = {}
            return
        self.gain32 = self.gain.to(torch.float32).contiguous()
        self._ones = {}
        if self.float32_stream or self.offset:
            self.as_gain = ops.Gain(self.gain.to(torch.float32).contiguous(), self.offset, self.eps, groups=self.groups)

    def stream_norm(self, streams: Optional[torch.Tensor], n_streams: int, *, start: Optional[torch.Tensor] = None,
                    y: Optional[torch.Tensor] = None, written=None, read: Optional[torch.Tensor] = None):
        """Over ``n_streams`` copies of the residual stream: the write of the sublayer that produced
        ``y`` (``written``: its :class:`ops.StreamNumbers`), then the read with the numbers ``read``
        (None: the sum of the copies) and this norm of it.  ``start``: the row every copy starts as.
        Returns (streams, normalised read)."""
        if read is None:
            if n_streams not in self._ones:
                self._ones[n_streams] = torch.ones(n_streams, dtype=torch.float32, device=self.gain32.device)
            read = self._ones[n_streams]
        return ops.hyper_norm(streams, n_streams, self.dtype, start=start, y=y, written=written, read=read,
                              gain=self.gain32, eps=self.eps)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.scalar_gain:
            return self.stream_norm(x, 1)[1]
        if self.float32_stream or self.offset:
            if x.dtype == torch.float32:
                return ops.residual_norm(x, None, None, self.as_gain, self.dtype)[1]
            # a stream that has not started yet: the rows are its first value
            return ops.residual_norm(None, x, None, self.as_gain, self.dtype)[1]
        return ops.rmsnorm(x, self.gain, self.eps)

    def start_forward(self, x: torch.Tensor):
        """``x`` of the activation type starts a float32 stream: returns (stream, norm of it)."""
        return ops.residual_norm(None, x, None, self.as_gain, self.dtype)

    def add_forward(self, h: torch.Tensor, d, post: Optional["RMSNorm"] = None) -> torch.Tensor:
        if isinstance(d, Branch):       # a branch with a second tensor or a factor (its norm comes as ``post``)
            if not self.float32_stream:
                raise ops.KernelError("rmsnorm: a branch of two tensors or with a factor needs a float32 stream")
            return ops.residual_norm(h, d.tensor, post.as_gain if post is not None else None, self.as_gain, self.dtype,
                                     d2=d.second, mult=d.factor)[1]
        if self.float32_stream:
            return ops.residual_norm(h, d, post.as_gain if post is not None else None, self.as_gain, self.dtype)[1]
        if post is not None or self.offset:
            raise ops.KernelError("rmsnorm: a norm of the branch before the add, or a gain offset, needs a float32 stream")
        return ops.add_rmsnorm(h, d, self.gain, self.eps)

    def add_only(self, h: torch.Tensor, d: torch.Tensor) -> None:
        """``h <- h + self(d)`` on a float32 stream, nothing else: this norm as the one a branch
        passes before the add, with no norm of the sum wanted."""
        ops.residual_norm(h, d, self.as_gain, None, self.dtype)


@register_part("norm", "layernorm")
class LayerNorm:
    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> List[TensorSpec]:
        size = int(spec.params["size"])
        specs = [TensorSpec(spec.tensors["weight"], (size,), GAIN)]
        if "bias" in spec.tensors:
            specs.append(TensorSpec(spec.tensors["bias"], (size,), GAIN, init="small_normal"))
        return specs

    def __init__(self, spec: PartSpec, runtime: Runtime):
        if spec.params.get("residual") != "float32":
            raise ValueError("layernorm: this norm works on a residual stream kept in float32 (residual: 'float32')")
        self.size = int(spec.params["size"])
        self.eps = float(spec.params["eps"])
        self.dtype = runtime.dtype
        bias = runtime.tensor(spec, "bias").to(torch.float32).contiguous() if "bias" in spec.tensors else None
        self.as_gain = ops.Gain(runtime.tensor(spec, "weight").to(torch.float32).contiguous(), 0.0, self.eps, bias, "layer")

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.residual_norm(x, None, None, self.as_gain, self.dtype)[1]

    def add_forward(self, h: torch.Tensor, d: torch.Tensor, post=None) -> torch.Tensor:
        return ops.residual_norm(h, d, post.as_gain if post is not None else None, self.as_gain, self.dtype)[1]

    def add_only(self, h: torch.Tensor, d: torch.Tensor) -> None:
        ops.residual_norm(h, d, self.as_gain, None, self.dtype)

    def read(self, h: torch.Tensor) -> torch.Tensor:
        """The stream rounded to the activation type: what a sublayer that reads the stream itself gets."""
        return ops.residual_norm(h, None, None, ops.STREAM_AS_IS, self.dtype)[1]

    def add_read(self, h: torch.Tensor, d: torch.Tensor) -> torch.Tensor:
        """``h <- h + self(d)``; returns the new stream rounded to the activation type."""
        return ops.residual_norm(h, d, self.as_gain, ops.STREAM_AS_IS, self.dtype)[1]
