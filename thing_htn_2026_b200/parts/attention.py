"""Grouped-query attention over the cache: the token mixer of this architecture.

One product gives q, k and v (weights concatenated ``[q; k; v]`` as the reference does,
engine/engine.py:214-216); one kernel normalises q and k per head, rotates them and writes
K and V to the cache (engine/kernels/torch_ref.py:107-162); attention then reads the
cache, which already holds the step's own keys (engine/kernels/torch_ref.py:168-227);
one product projects back (engine/engine.py:1114).

Parameters (all from the PartSpec): ``hidden_size, n_heads, n_kv_heads, head_dim, scale``,
``window`` (None: all keys; W: the last W keys), ``qk_norm_eps`` (None: no head norm) and
``position`` (a position PartSpec or None).  A schedule entry with ``writes_cache=False``
makes the mixer read the cache another entry wrote: it computes only its queries.

Further parameters, each with the first value as its default: ``qk_norm_scope`` "head" (an RMS
norm per head with gains ``[head_dim]``) or "projection" (one RMS norm over all heads of q and
one over all heads of k, before they are split into heads, with gains of those sizes);
``values`` "projection" (a value product of its own, ``v_proj``) or "keys" (the values are the
keys as projected, before norm and rotation: no ``v_proj``); ``keep_first`` 0 (with a window:
that many first positions of a sequence stay visible to every later query, at their own
positions).  The position part's ``layout`` chooses the pairs of the rotation.  Anything but
the defaults goes through :func:`ops.qk_prepare` (float32 inside, one rounding) instead of the
per-head kernel; ``prepare`` "float32" asks for that kernel with the defaults too.

``value_dim`` (default ``head_dim``): the size of a head's value where it differs from its
query's and key's.  ``chunk`` (instead of ``window``): position i sees j <= i only where
``floor(i / chunk) = floor(j / chunk)``, chunks counted from the sequence's first position.
``softmax_weights`` "float32": the weights stay float32 where they multiply the values, in
the kernels that do not put that product on tensor cores.

``softcap`` (a positive number): a score s becomes ``softcap * tanh(s / softcap)`` before the
softmax.  ``q_temp`` (a mapping ``coef, every``): the query at position p is multiplied by
``1 + coef * ln(floor((p + 1) / every) + 1)``; the kernels apply the factor to the row's scores in
float32.  ``kv`` "own" (default) or "shared": a "shared" mixer has no key and value projections
at all (no ``k_proj`` and ``v_proj`` tensors); every schedule entry that runs it reads the cache
that another layer wrote (``writes_cache=False``), with its own queries, scale, mask and score
shaping.
"""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import ops
from ..cache.sequence_cache import CacheNeed, KVSpec
from ..config.base import PartSpec, ScheduleEntry
from ..weights.loader import GAIN, MATRIX, TensorSpec
from .registry import part_class, register_part
from .runtime import HostBatch, Runtime, StepContext


@register_part("mixer", "attention")
class Attention:
    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> List[TensorSpec]:
        p = spec.params
        hidden, n_q, n_kv, d = int(p["hidden_size"]), int(p["n_heads"]), int(p["n_kv_heads"]), int(p["head_dim"])
        dv = int(p.get("value_dim") or d)
        specs = [TensorSpec(spec.tensors["q_proj"], (n_q * d, hidden), MATRIX)]
        if p.get("kv", "own") != "shared":
            specs.append(TensorSpec(spec.tensors["k_proj"], (n_kv * d, hidden), MATRIX))
            if p.get("values", "projection") == "projection":
                specs.append(TensorSpec(spec.tensors["v_proj"], (n_kv * dv, hidden), MATRIX))
        specs.append(TensorSpec(spec.tensors["o_proj"], (hidden, n_q * dv), MATRIX))
        if p.get("qk_norm_eps") is not None:
            whole = p.get("qk_norm_scope", "head") == "projection"
            specs += [TensorSpec(spec.tensors["q_norm"], (n_q * d if whole else d,), GAIN),
                      TensorSpec(spec.tensors["k_norm"], (n_kv * d if whole else d,), GAIN)]
        return specs

    def __init__(self, spec: PartSpec, runtime: Runtime):
        p = spec.params
        self.n_q, self.n_kv, self.head_dim = int(p["n_heads"]), int(p["n_kv_heads"]), int(p["head_dim"])
        if self.n_q % self.n_kv:
            raise ValueError(f"attention: {self.n_q} heads are not a multiple of {self.n_kv} kv heads")
        self.scale = float(p["scale"])
        self.value_dim = int(p.get("value_dim") or self.head_dim)
        self.chunk: Optional[int] = None if p.get("chunk") is None else int(p["chunk"])
        if self.chunk is not None and (self.chunk <= 0 or p.get("window") is not None):
            raise ValueError("attention: a chunk size is positive and stands instead of a window")
        self.exact_weights = p.get("softmax_weights") == "float32"
        self.window: Optional[int] = None if p.get("window") is None else int(p["window"])
        self.eps = None if p.get("qk_norm_eps") is None else float(p["qk_norm_eps"])
        self.keep_first = int(p.get("keep_first") or 0) if self.window else 0
        self.norm_scope = str(p.get("qk_norm_scope", "head")) if self.eps is not None else None
        self.values_are_keys = p.get("values", "projection") == "keys"
        if self.norm_scope not in (None, "head", "projection") or p.get("values", "projection") not in ("projection", "keys"):
            raise ValueError(f"attention: qk_norm_scope {p.get('qk_norm_scope')!r} or values {p.get('values')!r} unknown")
        if self.values_are_keys and self.value_dim != self.head_dim:
            raise ValueError("attention: values that are the keys have the keys' size")
        if p.get("kv", "own") not in ("own", "shared"):
            raise ValueError(f"attention: kv {p.get('kv')!r} is neither 'own' nor 'shared'")
        self.shared_kv = p.get("kv", "own") == "shared"
        if self.shared_kv and (p.get("qk_norm_eps") is not None or p.get("position") is not None):
            raise ValueError("attention: a mixer without keys of its own has no q/k norm and no rotation here")
        projections = [runtime.tensor(spec, "q_proj")]
        if not self.shared_kv:
            projections.append(runtime.tensor(spec, "k_proj"))
            if not self.values_are_keys:
                projections.append(runtime.tensor(spec, "v_proj"))
        self.w_qkv = torch.cat(projections, dim=0).contiguous() if len(projections) > 1 else projections[0]
        temp = p.get("q_temp")
        self.shape = ops.ScoreShape(float(p.get("softcap") or 0.0), float(temp["coef"]) if temp else 0.0,
                                    int(temp["every"]) if temp else 0)
        if self.shape.softcap < 0 or self.shape.temp_every < 0:
            raise ValueError("attention: softcap and q_temp.every are positive")
        self.w_o = runtime.tensor(spec, "o_proj")
        self.q_gain = runtime.tensor(spec, "q_norm") if self.eps is not None else None
        self.k_gain = runtime.tensor(spec, "k_norm") if self.eps is not None else None
        self.dtype = runtime.dtype
        self.position = None
        position_spec = p.get("position")
        if position_spec is not None:
            key = "position:" + position_spec.key()
            if key not in runtime.shared:
                runtime.shared[key] = part_class("position", position_spec.kind)(position_spec, runtime)
            self.position = runtime.shared[key]
        # The per-head kernel (and the kernel that fuses it with single-token attention) takes the
        # defaults; every other variant is prepared by the general kernel.
        self.general = (self.norm_scope == "projection" or self.values_are_keys
                        or p.get("prepare") == "float32" or self.value_dim != self.head_dim
                        or (self.position is not None and getattr(self.position, "layout", "half") != "half"))
        if self.general and self.eps is not None:
            self.q_gain, self.k_gain = self.q_gain.float().contiguous(), self.k_gain.float().contiguous()

    def cache_need(self) -> CacheNeed:
        if self.shared_kv:
            return None
        return KVSpec(self.n_kv, self.head_dim, self.window, self.keep_first, self.chunk, self.value_dim)

    def _tile(self, page_size: int) -> int:
        return ops.prompt_attention_tile(self.dtype, self.head_dim, page_size, self.n_q, self.n_kv, self.value_dim,
                                         self.chunk)

    def step_inputs(self, batch: HostBatch, out: Dict[str, List[int]]) -> None:
        """The prompt attention kernels work on tiles of consecutive rows of one sequence; the
        host knows every length, so it lists them (every attention of a model that wants
        tiles of one size shares one list)."""
        size = self._tile(batch.page_size) if batch.max_count > 1 else 0
        if size and f"row_tiles/{size}/row0" not in out:
            out[f"row_tiles/{size}/row0"], out[f"row_tiles/{size}/rows"] = ops.row_tiles_of(
                batch.counts, batch.held, size)

    def forward(self, x: torch.Tensor, ctx: StepContext, entry: ScheduleEntry) -> torch.Tensor:
        kv = ctx.cache.kv_view(entry.cache)
        tiles = None
        if ctx.rows.max_q_len > 1:
            size = self._tile(kv.page_size)
            row0 = ctx.inputs.get(f"row_tiles/{size}/row0") if size else None
            if row0 is not None:
                tiles = ops.RowTiles(row0, ctx.inputs[f"row_tiles/{size}/rows"], row0.shape[0], size)
        qkv = ops.linear(x, self.w_qkv, err=ctx.err)
        if self.shared_kv:
            if entry.writes_cache:
                raise ValueError("attention: a mixer without keys of its own cannot write a cache")
            # the projected rows are the queries: nothing to normalise, rotate or store
            a = ops.attention(qkv, ctx.rows, kv, self.n_q, self.scale, self.window, ctx.err, tiles, self.keep_first,
                              self.chunk, self.exact_weights, self.shape)
            return ops.linear(a, self.w_o, err=ctx.err)
        if self.general or self.keep_first or self.chunk or self.exact_weights or self.shape.active:
            rotary = self.position.tables() if self.position is not None else None
            if self.general:
                q = ops.qk_prepare(qkv, self.q_gain, self.k_gain, self.norm_scope, self.eps or 1.0, rotary, ctx.rows, kv,
                                   self.n_q, self.values_are_keys, entry.writes_cache, ctx.err)
            else:
                q = ops.qk_norm_rope_cache(qkv, self.q_gain, self.k_gain, self.eps if self.eps is not None else 1.0,
                                           rotary, ctx.rows, kv, self.n_q, entry.writes_cache, ctx.err)
            a = ops.attention(q, ctx.rows, kv, self.n_q, self.scale, self.window, ctx.err, tiles, self.keep_first,
                              self.chunk, self.exact_weights, self.shape)
            return ops.linear(a, self.w_o, err=ctx.err)
        a = ops.qkv_attention(qkv, self.q_gain, self.k_gain, self.eps if self.eps is not None else 1.0,
                              self.position.tables() if self.position is not None else None,
                              ctx.rows, kv, self.n_q, self.scale, self.window, entry.writes_cache, ctx.err, tiles)
        return ops.linear(a, self.w_o, err=ctx.err)
