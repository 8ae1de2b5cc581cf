"""Token embedding (a row gather, engine/engine.py:1101) and the LM head
(engine/engine.py:1120; with tied weights it is the embedding table, :225-226).
Logits are float32.

The embedding takes two optional parameters: ``scale`` (the rows are multiplied by it) and
``stream`` "float32" (the rows come out in float32, scaled in float32: the start of a residual
stream that is kept in float32).  ``positions`` (a mapping ``kind: "sinusoid", base``; float32
stream only): a position vector is added to every row, ``sin(p w_i)`` at entry 2i and
``cos(p w_i)`` at entry 2i + 1 with ``w_i = base^(-2i / hidden_size)`` and p the row's position
in its sequence; the frequencies are computed in double on the host, the angles and their sines
in double on the device.

The head takes ``scale`` (default 1): a constant factor on the logits."""

from __future__ import annotations

from typing import List, Optional

import torch

from .. import ops
from ..config.base import PartSpec
from ..weights.loader import MATRIX, TensorSpec
from .registry import register_part
from .runtime import Runtime


@register_part("embedding", "embedding")
class Embedding:
    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> List[TensorSpec]:
        return [TensorSpec(spec.tensors["weight"], (int(spec.params["vocab_size"]), int(spec.params["hidden_size"])),
                           MATRIX)]

    def __init__(self, spec: PartSpec, runtime: Runtime):
        self.table = runtime.tensor(spec, "weight")
        self.scale = float(spec.params.get("scale", 1.0))
        self.float32_stream = spec.params.get("stream") == "float32"
        if self.scale != 1.0 and not self.float32_stream:
            raise ValueError("embedding: a scale needs stream 'float32'")
        self.frequencies = None
        positions = spec.params.get("positions")
        if positions is not None:
            if positions.get("kind") != "sinusoid" or not self.float32_stream:
                raise ValueError("embedding: positions are of kind 'sinusoid' and need stream 'float32'")
            width = int(spec.params["hidden_size"])
            pair = torch.arange((width + 1) // 2, dtype=torch.float64)
            self.frequencies = (float(positions["base"]) ** (-2.0 * pair / width)).to(runtime.device)

    def forward(self, tokens: torch.Tensor, err: torch.Tensor, rows: Optional[ops.StepRows] = None) -> torch.Tensor:
        """``rows``: the step's rows, for an embedding that adds positions."""
        if self.frequencies is not None:
            if rows is None:
                raise ValueError("embedding: positions are added, the step's rows are needed")
            return ops.gather_rows_scaled(self.table, tokens, self.scale, err, rows.row_pos, self.frequencies)
        if self.float32_stream:
            return ops.gather_rows_scaled(self.table, tokens, self.scale, err)
        return ops.gather_rows(self.table, tokens, err)


@register_part("head", "lm_head")
class LMHead:
    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> List[TensorSpec]:
        copies = (spec.tensors["stored_copy"],) if "stored_copy" in spec.tensors else ()
        return [TensorSpec(spec.tensors["weight"], (int(spec.params["vocab_size"]), int(spec.params["hidden_size"])),
                           MATRIX, copies=copies)]

    def __init__(self, spec: PartSpec, runtime: Runtime):
        self.weight = runtime.tensor(spec, "weight")
        self.vocab_size = int(spec.params["vocab_size"])
        self.scale = float(spec.params.get("scale", 1.0))

    def forward(self, x: torch.Tensor, err: Optional[torch.Tensor] = None) -> torch.Tensor:
        logits = ops.linear(x, self.weight, out_dtype=torch.float32, err=err)
        return ops.scale_(logits, self.scale) if self.scale != 1.0 else logits
