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
``h <- h + factor * (d + d')``.

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
        return [TensorSpec(spec.tensors["weight"], (int(spec.params["size"]),), GAIN, init=init)]

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
        if self.float32_stream or self.offset:
            self.as_gain = ops.Gain(self.gain.to(torch.float32).contiguous(), self.offset, self.eps, groups=self.groups)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
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
