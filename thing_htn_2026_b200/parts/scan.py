"""The selective scan (Mamba): a recurrent token mixer with a state vector per channel.

    [x | z] = W_in h                                   (``inner`` channels each)
    x <- silu(conv(x) + b_conv)                        (a causal convolution per channel over ``conv_taps``
                                                        tokens, the last tap the current token's, zeros before the start)
    [dt | B | C] = W_x x                               (``dt_rank``, ``state``, ``state`` entries)
    dt <- softplus(W_dt dt + b_dt)                     (one step size per channel)
    S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n,   A = -exp(A_log)
    y_c = sum_n S[c, n] C_n + D_c x_c;   out = W_o (y * silu(z))

State per sequence, zero when a slot opens: ``S`` float32 ``[inner, state]`` and a ring of the last
``conv_taps`` raw inputs of the convolution (position p at ``p mod conv_taps``).  The step size with
its softplus, the decay with its exponential, the state and the sums are float32; the projection to
the step size keeps its float32 result.  ``W_x`` is held as two weights (the ``dt`` rows, filled up
with zero rows to a multiple of eight, and the ``B``, ``C`` rows), so that each product's result is
what the next kernel reads.  Kernels: csrc/selective_scan.cu.
"""

from __future__ import annotations

from typing import List

import torch

from .. import ops
from ..cache.sequence_cache import CacheNeed, StateSpec
from ..config.base import PartSpec, ScheduleEntry
from ..weights.loader import GAIN, MATRIX, TensorSpec
from .linear_attention import pad_rank
from .registry import register_part
from .runtime import Runtime, StepContext


@register_part("mixer", "selective_scan")
class SelectiveScan:
    @staticmethod
    def _sizes(spec: PartSpec):
        p = spec.params
        return int(p["hidden_size"]), int(p["inner"]), int(p["state"]), int(p["dt_rank"]), int(p["conv_taps"])

    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> List[TensorSpec]:
        hidden, inner, n, r, taps = cls._sizes(spec)
        t = spec.tensors
        return [TensorSpec(t["in"], (2 * inner, hidden), MATRIX),
                TensorSpec(t["conv"], (inner, taps), GAIN, init="conv_taps"),
                TensorSpec(t["conv_bias"], (inner,), GAIN, init="small_normal"),
                TensorSpec(t["x"], (r + 2 * n, inner), MATRIX),
                TensorSpec(t["dt"], (inner, r), MATRIX, init="unit_normal"),
                TensorSpec(t["dt_bias"], (inner,), GAIN, init="small_normal"),
                TensorSpec(t["A_log"], (inner, n), GAIN, init="log_spread"),
                TensorSpec(t["D"], (inner,), GAIN),
                TensorSpec(t["o"], (hidden, inner), MATRIX)]

    def __init__(self, spec: PartSpec, runtime: Runtime):
        _, self.inner, self.n_state, self.dt_rank, self.taps = self._sizes(spec)
        self.dtype = runtime.dtype
        f32 = lambda t: t.to(torch.float32).contiguous()
        self.w_in = runtime.tensor(spec, "in")
        self.w_o = runtime.tensor(spec, "o")
        w_x = runtime.tensor(spec, "x")
        self.w_bc = w_x[self.dt_rank:].contiguous()
        w_low, self.w_dt = pad_rank(w_x[:self.dt_rank], runtime.tensor(spec, "dt"))
        self.w_low = w_low
        self.conv_w, self.conv_b = f32(runtime.tensor(spec, "conv")), f32(runtime.tensor(spec, "conv_bias"))
        self.dt_bias = f32(runtime.tensor(spec, "dt_bias"))
        self.a = (-torch.exp(runtime.tensor(spec, "A_log").to(torch.float64))).to(torch.float32).contiguous()
        self.d = f32(runtime.tensor(spec, "D"))

    def cache_need(self) -> CacheNeed:
        return (StateSpec((self.inner, self.n_state), torch.float32), StateSpec((self.taps, self.inner), self.dtype))

    def forward(self, x: torch.Tensor, ctx: StepContext, entry: ScheduleEntry) -> torch.Tensor:
        state, ring = ctx.cache.state_view(entry.cache, 0), ctx.cache.state_view(entry.cache, 1)
        proj = ops.linear(x, self.w_in, err=ctx.err)
        xc = ops.causal_conv(proj, 0, self.inner, self.conv_w, self.conv_b, ring, ctx.rows, ctx.cache.seq_lens)
        ops.conv_ring_update(ring, proj, 0, ctx.rows, ctx.cache.seq_lens)
        bc = ops.linear(xc, self.w_bc, err=ctx.err)
        dt = ops.linear(ops.linear(xc, self.w_low, err=ctx.err), self.w_dt, out_dtype=torch.float32, err=ctx.err)
        y = ops.selective_scan(xc, dt, self.dt_bias, bc, self.a, self.d, proj, self.inner, state, ctx.rows)
        return ops.linear(y, self.w_o, err=ctx.err)
