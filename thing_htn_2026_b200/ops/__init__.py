"""Python faces of the CUDA kernels.  Every function here takes CUDA tensors and launches
on the current stream; there is no CPU path.  Matrix products of the bfloat16 path may
go to the vendor library, as the reference's do (engine/engine.py:341-350); everything
else, and every product of the 32-bit path, is this library's own kernel.
"""

from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch

from . import library
from .library import KernelLibraryError

c_int, c_float, c_void_p, c_longlong = ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_longlong

DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}

# device error word bits (csrc/common.cuh)
ERR_TOKEN_RANGE, ERR_PAGE_UNMAPPED, ERR_POSITION_RANGE, ERR_WAIT_TIMEOUT = 1, 2, 4, 8
_ERR_TEXT = {
    ERR_TOKEN_RANGE: "a token id outside the vocabulary",
    ERR_PAGE_UNMAPPED: "a cache position whose page is not mapped",
    ERR_POSITION_RANGE: "a position beyond the rotary table",
    ERR_WAIT_TIMEOUT: "a bounded wait inside a kernel gave up",
}


class KernelError(RuntimeError):
    """A launcher refused its arguments, or a kernel reported a fault."""


_SIGNATURES = {
    "thn_gather_rows": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "thn_rmsnorm": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_int, c_void_p],
    "thn_swiglu": [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "thn_gemm_tcgen05_supported": [c_int, c_int, c_int],
    "thn_gemm_tcgen05_bf16": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "thn_gemm_stream_supported": [c_int, c_int, c_int],
    "thn_gemm_stream_scratch": [c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "thn_gemm_stream_bf16": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                             c_int, c_void_p, c_void_p],
    "thn_step_rows": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p],
    "thn_advance": [c_void_p, c_void_p, c_void_p, c_int, c_void_p],
    "thn_rope_table": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "thn_qk_norm_rope_cache": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_float, c_void_p, c_void_p, c_int,
                               c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                               c_int, c_int, c_int, c_void_p, c_void_p],
    "thn_attention_decode_fused_bf16": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_float, c_void_p, c_void_p, c_int,
                                        c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                        c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p, c_longlong, c_int,
                                        c_void_p, c_void_p],
    "thn_attention_generic": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                              c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int, c_int, c_float, c_float, c_int,
                              c_void_p, c_int, c_void_p, c_void_p],
    "thn_residual_norm": [c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_float, c_float, c_int,
                          c_void_p, c_void_p, c_float, c_float, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "thn_gated_head_norm": [c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_float, c_int, c_int, c_int, c_int,
                            c_int, c_longlong, c_float, c_int, c_void_p],
    "thn_hyper_norm": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_float,
                       c_int, c_int, c_int, c_int, c_void_p],
    "thn_linear_attention": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int,
                             c_void_p, c_float, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int,
                             c_int, c_void_p],
    "thn_causal_conv": [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                        c_int, c_int, c_int, c_int, c_void_p],
    "thn_conv_ring_update": [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                             c_void_p],
    "thn_selective_scan": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                           c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "thn_rotate_gate": [c_void_p, c_longlong, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_int, c_int,
                        c_void_p, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p],
    "thn_add_bias_f32": [c_void_p, c_void_p, c_int, c_int, c_float, c_void_p],
    "thn_gather_rows_scaled": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p, c_void_p, c_int,
                               c_void_p, c_void_p],
    "thn_scale_f32": [c_void_p, c_longlong, c_float, c_void_p],
    "thn_polynorm": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_void_p],
    "thn_routed_clamped_glu": [c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_float,
                               c_float, c_float, c_int, c_int, c_void_p],
    "thn_logistic_gate": [c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_void_p],
    "thn_latent_norm": [c_void_p, c_void_p, c_longlong, c_void_p, c_float, c_int, c_int, c_int, c_void_p],
    "thn_latent_assemble": [c_void_p, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int,
                            c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                            c_int, c_void_p, c_void_p],
    "thn_mlstm_columns_per_block": [],
    "thn_mlstm_gates": [c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_int, c_int, c_void_p],
    "thn_mlstm_recurrence": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_float, c_int,
                             c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_float, c_int, c_void_p],
    "thn_moe_route": [c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_int, c_float,
                      c_int, c_int, c_float, c_void_p],
    "thn_routed_gelu": [c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "thn_clamped_glu": [c_void_p, c_void_p, c_int, c_int, c_float, c_float, c_int, c_void_p],
    "thn_qk_prepare": [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_float, c_float, c_void_p, c_void_p,
                       c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                       c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p],
    "thn_delta_prepare": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                          c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                          c_float, c_int, c_void_p],
    "thn_delta_recurrence": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                             c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "thn_delta_conv_ring_update": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                   c_int, c_int, c_int, c_void_p],
    "thn_delta_decode": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                         c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p],
    "thn_gemm_f32": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "thn_linear_skinny_bf16": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "thn_linear_skinny_supported": [c_int, c_int],
    "thn_scatter_i32": [c_void_p, c_void_p, c_void_p, c_int, c_longlong, c_void_p],
    "thn_choose_tokens": [c_void_p, c_void_p, c_int, c_int, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p,
                          c_void_p, c_void_p, c_int, c_void_p, c_void_p],
    "thn_gather_i32": [c_void_p, c_void_p, c_void_p, c_int, c_void_p],
    "thn_attention_mma_supported": [c_int, c_int, c_int, c_int],
    "thn_attention_fused_supported": [c_int, c_int, c_int, c_int],
    "thn_attention_prefill_bf16": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                   c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int, c_int,
                                   c_float, c_float, c_int, c_void_p, c_void_p, c_void_p],
    "thn_attention_decode_bf16": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                  c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int, c_int, c_float, c_float,
                                  c_int, c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_void_p, c_void_p],
    "thn_attention_decode_blocks_per_sm": [c_int],
    "thn_attention_decode_cluster_splits": [],
    "thn_attention_decode_one_wave_splits": [c_int, c_int, c_int],
    "thn_attention_prefill_tile_rows": [],
    "thn_attention_decode_last_variant": [],
    "thn_attention_decode_streams": [],
    "thn_attention_tcgen05_supported": [c_int, c_int, c_int, c_int],
    "thn_attention_tcgen05_test_skip_loads": [c_int],
    "thn_attention_prefill_tcgen05": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p,
                                      c_void_p, c_longlong, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float,
                                      c_int, c_int, c_int, c_float, c_float, c_int, c_void_p, c_void_p, c_void_p],
}

_lib = None


def lib():
    global _lib
    if _lib is None:
        loaded = library.load()
        for name, argtypes in _SIGNATURES.items():
            fn = getattr(loaded, name)
            fn.argtypes = argtypes
            fn.restype = c_int
        loaded.thn_set_pdl.argtypes = [c_int]
        loaded.thn_set_pdl.restype = None
        loaded.thn_set_pdl(0 if os.environ.get("THN_PDL", "1").strip().lower() in ("0", "false", "no", "off") else 1)
        loaded.thn_set_stream_early.argtypes = [c_int]
        loaded.thn_set_stream_early.restype = None
        if os.environ.get("THN_STREAM_EARLY"):
            loaded.thn_set_stream_early(int(os.environ["THN_STREAM_EARLY"]))
        loaded.thn_set_decode_cluster.argtypes = [c_int]
        loaded.thn_set_decode_cluster.restype = None
        loaded.thn_set_decode_cluster(0 if os.environ.get("THN_DECODE_CLUSTER", "1").strip() in ("0", "false", "off") else 1)
        loaded.thn_set_decode_stream_order.argtypes = [c_int]
        loaded.thn_set_decode_stream_order.restype = None
        loaded.thn_set_decode_stream_order(int(os.environ.get("THN_DECODE_STREAM_BY_LENGTH", 1)))
        loaded.thn_set_decode_stream.argtypes = [c_int, c_int]
        loaded.thn_set_decode_stream.restype = None
        loaded.thn_set_decode_stream(int(os.environ.get("THN_DECODE_STREAM", 1)),
                                     int(os.environ.get("THN_DECODE_STREAM_STAGES", 3)))
        loaded.thn_set_mlstm_staged.argtypes = [c_int, c_int]
        loaded.thn_set_mlstm_staged.restype = None
        loaded.thn_set_mlstm_staged(0 if os.environ.get("THN_MLSTM_STAGED", "1").strip() in ("0", "false", "off") else 1,
                                    int(os.environ.get("THN_MLSTM_LANES", 0)))
        loaded.thn_choose_tokens_scratch_floats.argtypes = [c_int, c_int]
        loaded.thn_choose_tokens_scratch_floats.restype = c_longlong
        loaded.thn_attention_decode_scratch_floats.argtypes = [c_int, c_int, c_int, c_int]
        loaded.thn_attention_decode_scratch_floats.restype = c_longlong
        loaded.thn_linear_attention_scratch_floats.argtypes = [c_int, c_int, c_int, c_int, c_int]
        loaded.thn_linear_attention_scratch_floats.restype = c_longlong
        _lib = loaded
    return _lib


_sm_count = {}
launch_count = 0   # kernels of this library launched (or recorded into a graph) so far
calls_by_entry: Dict[str, int] = {}    # the same, per entry point of the kernel library


def _call(name: str, *args) -> None:
    global launch_count
    launch_count += 1
    calls_by_entry[name] = calls_by_entry.get(name, 0) + 1
    code = getattr(lib(), name)(*args)
    if code:
        raise KernelError(f"{name}: {lib().thn_last_error().decode()} (status {code})")


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _need(t: torch.Tensor, what: str, dtype=None) -> torch.Tensor:
    if not t.is_cuda:
        raise KernelError(f"{what}: tensor is on {t.device}; this library runs on CUDA only")
    if not t.is_contiguous():
        raise KernelError(f"{what}: tensor must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{what}: expected {dtype}, got {t.dtype}")
    return t


def _code(t: torch.Tensor, what: str) -> int:
    try:
        return DTYPE_CODE[t.dtype]
    except KeyError:
        raise KernelError(f"{what}: dtype {t.dtype} is not supported (float32 or bfloat16)") from None


def new_error_word(device) -> torch.Tensor:
    return torch.zeros(1, dtype=torch.int32, device=device)


def raise_on_device_error(err: torch.Tensor, where: str) -> None:
    """Reads the error word (a synchronising copy) and raises if a kernel set a bit."""
    bits = int(err.item())
    if bits:
        err.zero_()
        reasons = [text for bit, text in _ERR_TEXT.items() if bits & bit]
        raise KernelError(f"{where}: device reported " + "; ".join(reasons))


# ------------------------------------------------------------------ rows and lengths


@dataclass
class StepRows:
    """Per-row indices of a packed step: the slot of each row's sequence and the row's
    absolute position; plus the batch description they were made from."""

    row_slot: torch.Tensor   # int32 [rows]
    row_pos: torch.Tensor    # int32 [rows]
    slots: torch.Tensor      # int32 [seqs]
    cu_seqlens: torch.Tensor  # int32 [seqs + 1]
    n_rows: int
    n_seqs: int
    max_q_len: int           # longest run of rows of one sequence (host knowledge)
    # Host knowledge: the most keys a row of this step may see (an upper bound; None: unknown).
    # Kernels may divide their work by it, which changes a result by rounding at most.  A step
    # captured as a graph is replayed only while its bound holds (see context_class).
    max_context: Optional[int] = None
    # Host knowledge: False if the sequences of the step hold about the same number of keys (see
    # lengths_differ); None: unknown.  Like max_context a hint that changes no result.
    lengths_differ: Optional[bool] = None


LONG_CONTEXT = 8192     # keys; a single-token step of few long sequences divides each key range further
CONTEXT_CLASS_BASE = 1024   # keys; the first class of context length ends below it
STREAM_MIN_CONTEXT = 1024   # keys from which many unsplit sequences go to the streaming decode attention


def context_class(longest: int) -> Tuple[int, int]:
    """(class, bound) of a step whose longest sequence holds ``longest`` keys: class 0 below
    CONTEXT_CLASS_BASE, then one class per doubling.  Steps of one class make the same choices,
    so one captured graph serves them; ``bound`` is the class's ``max_context``."""
    k = (max(0, int(longest)) // CONTEXT_CLASS_BASE).bit_length()
    return k, (CONTEXT_CLASS_BASE << k) - 1


def lengths_differ(lengths) -> bool:
    """Whether the shortest of the sequences is more than a quarter shorter than the longest:
    the class of a step, beside ``context_class``, by which a captured graph is chosen."""
    longest = max(lengths)
    return (longest - min(lengths)) * 4 > longest


def step_rows(cu_seqlens: torch.Tensor, slots: torch.Tensor, seq_lens: torch.Tensor, n_rows: int,
              max_q_len: int, out: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
              max_context: Optional[int] = None, lengths_differ: Optional[bool] = None) -> StepRows:
    _need(cu_seqlens, "step_rows cu_seqlens", torch.int32)
    _need(slots, "step_rows slots", torch.int32)
    _need(seq_lens, "step_rows seq_lens", torch.int32)
    n_seqs = slots.shape[0]
    if out is None:
        row_slot = torch.empty(n_rows, dtype=torch.int32, device=slots.device)
        row_pos = torch.empty(n_rows, dtype=torch.int32, device=slots.device)
    else:
        row_slot, row_pos = out
    _call("thn_step_rows", _ptr(row_slot), _ptr(row_pos), _ptr(cu_seqlens), _ptr(slots), _ptr(seq_lens), n_seqs,
          _stream())
    return StepRows(row_slot, row_pos, slots, cu_seqlens, n_rows, n_seqs, max_q_len, max_context=max_context,
                    lengths_differ=lengths_differ)


def advance(seq_lens: torch.Tensor, slots: torch.Tensor, cu_seqlens: torch.Tensor) -> None:
    _call("thn_advance", _ptr(_need(seq_lens, "advance seq_lens", torch.int32)), _ptr(slots), _ptr(cu_seqlens),
          slots.shape[0], _stream())


def scatter_i32(dst: torch.Tensor, index: torch.Tensor, value: torch.Tensor) -> None:
    """dst.view(-1)[index[i]] = value[i]; index int64, value int32, all on the device."""
    _need(dst, "scatter_i32 dst", torch.int32)
    _need(index, "scatter_i32 index", torch.int64)
    _need(value, "scatter_i32 value", torch.int32)
    _call("thn_scatter_i32", _ptr(dst), _ptr(index), _ptr(value), index.shape[0], dst.numel(), _stream())


# ------------------------------------------------------------------ elementwise


def gather_rows(table: torch.Tensor, index: torch.Tensor, err: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[m] = table[index[m]]; an index outside the table sets ERR_TOKEN_RANGE."""
    _need(table, "gather_rows table")
    _need(index, "gather_rows index", torch.int32)
    out = torch.empty((index.shape[0], table.shape[1]), dtype=table.dtype, device=table.device)
    _call("thn_gather_rows", _ptr(out), _ptr(table), _ptr(index), index.shape[0], table.shape[1], table.shape[0],
          _code(table, "gather_rows"), _ptr(err), _stream())
    return out


def gather_rows_scaled(table: torch.Tensor, index: torch.Tensor, scale: float,
                       err: Optional[torch.Tensor] = None, row_pos: Optional[torch.Tensor] = None,
                       frequencies: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[m] = float32(table[index[m]]) * scale: rows that start a residual stream kept in float32.
    With ``frequencies`` (float64 [ceil(width / 2)]) and ``row_pos`` (int32 [rows]) a sinusoidal
    position vector is added: ``sin(p f_i)`` at entry 2i and ``cos(p f_i)`` at entry 2i + 1."""
    _need(table, "gather_rows_scaled table")
    _need(index, "gather_rows_scaled index", torch.int32)
    if (row_pos is None) != (frequencies is None):
        raise KernelError("gather_rows_scaled: positions and frequencies go together")
    if frequencies is not None:
        _need(frequencies, "gather_rows_scaled frequencies", torch.float64)
        _need(row_pos, "gather_rows_scaled positions", torch.int32)
        if frequencies.shape[0] != (table.shape[1] + 1) // 2 or row_pos.shape[0] != index.shape[0]:
            raise KernelError(f"gather_rows_scaled: {frequencies.shape[0]} frequencies for rows of {table.shape[1]}, "
                              f"{row_pos.shape[0]} positions for {index.shape[0]} rows")
    out = torch.empty((index.shape[0], table.shape[1]), dtype=torch.float32, device=table.device)
    _call("thn_gather_rows_scaled", _ptr(out), _ptr(table), _ptr(index), index.shape[0], table.shape[1], table.shape[0],
          float(scale), _ptr(row_pos), _ptr(frequencies), _code(table, "gather_rows_scaled"), _ptr(err), _stream())
    return out


def scale_(x: torch.Tensor, scale: float) -> torch.Tensor:
    """x *= scale in place (float32): a constant factor on logits."""
    _need(x, "scale_", torch.float32)
    if scale != 1.0:
        _call("thn_scale_f32", _ptr(x), x.numel(), float(scale), _stream())
    return x


def polynorm(z: torch.Tensor, coefficients: torch.Tensor, eps: float) -> torch.Tensor:
    """z [rows, width] -> ``a N(z) + b N(z^2) + c N(z^3) + e`` with powers taken entry by entry,
    ``N(v) = v / sqrt(mean(v^2) + eps)`` over a row and ``(a, b, c, e) = coefficients`` (float32 [4])."""
    _need(z, "polynorm z")
    _need(coefficients, "polynorm coefficients", torch.float32)
    if z.dim() != 2 or coefficients.numel() != 4:
        raise KernelError(f"polynorm: shapes z {tuple(z.shape)}, coefficients {tuple(coefficients.shape)}")
    out = torch.empty_like(z)
    _call("thn_polynorm", _ptr(out), _ptr(z), _ptr(coefficients), z.shape[0], z.shape[1], float(eps), _code(z, "polynorm"),
          _stream())
    return out


def logistic_gate(a: torch.Tensor, gate: torch.Tensor, gate_offset: int = 0) -> torch.Tensor:
    """a [rows, width] * logistic(gate[:, gate_offset : gate_offset + width]); the gate may be a
    slice of a wider projected row."""
    _need(a, "logistic_gate a")
    _need(gate, "logistic_gate gate", a.dtype)
    rows, width = a.shape
    if gate.shape[0] != rows or gate_offset + width > gate.shape[1]:
        raise KernelError(f"logistic_gate: shapes a {tuple(a.shape)}, gate {tuple(gate.shape)} from column {gate_offset}")
    out = torch.empty_like(a)
    _call("thn_logistic_gate", _ptr(out), _ptr(a), gate.data_ptr() + gate_offset * gate.element_size(), gate.shape[1],
          rows, width, _code(a, "logistic_gate"), _stream())
    return out


def rmsnorm(x: torch.Tensor, gain: torch.Tensor, eps: float) -> torch.Tensor:
    _need(x, "rmsnorm x")
    _need(gain, "rmsnorm gain")
    if gain.shape[0] != x.shape[-1]:
        raise KernelError(f"rmsnorm: gain has {gain.shape[0]} entries, rows have {x.shape[-1]}")
    y = torch.empty_like(x)
    rows = x.numel() // x.shape[-1]
    _call("thn_rmsnorm", _ptr(y), _ptr(x), None, _ptr(gain), rows, x.shape[-1], float(eps),
          _code(x, "rmsnorm"), _code(gain, "rmsnorm gain"), _stream())
    return y


def add_rmsnorm(h: torch.Tensor, d: torch.Tensor, gain: torch.Tensor, eps: float) -> torch.Tensor:
    """h <- round(h + d) in place; returns RMSNorm(h) * gain."""
    _need(h, "add_rmsnorm h")
    _need(d, "add_rmsnorm d", h.dtype)
    _need(gain, "add_rmsnorm gain")
    if tuple(d.shape) != tuple(h.shape) or gain.shape[0] != h.shape[-1]:
        raise KernelError(f"add_rmsnorm: shapes h {tuple(h.shape)}, d {tuple(d.shape)}, gain {tuple(gain.shape)}")
    y = torch.empty_like(h)
    rows = h.numel() // h.shape[-1]
    _call("thn_rmsnorm", _ptr(y), _ptr(h), _ptr(d), _ptr(gain), rows, h.shape[-1], float(eps),
          _code(h, "add_rmsnorm"), _code(gain, "add_rmsnorm gain"), _stream())
    return y


def swiglu(gu: torch.Tensor) -> torch.Tensor:
    """gu [rows, 2*I] (gate columns first) -> silu(gate) * up, [rows, I]."""
    _need(gu, "swiglu")
    rows, width = gu.shape
    if width % 2:
        raise KernelError(f"swiglu: width {width} is odd")
    out = torch.empty((rows, width // 2), dtype=gu.dtype, device=gu.device)
    _call("thn_swiglu", _ptr(out), _ptr(gu), rows, width // 2, _code(gu, "swiglu"), _stream())
    return out


def clamped_glu(gu: torch.Tensor, limit: float, alpha: float) -> torch.Tensor:
    """gu [rows, 2*I] (gate columns first) -> g * logistic(alpha * g) * (u + 1) with
    g = min(gate, limit) and u = clamp(up, -limit, limit), [rows, I]."""
    _need(gu, "clamped_glu")
    rows, width = gu.shape
    if width % 2:
        raise KernelError(f"clamped_glu: width {width} is odd")
    out = torch.empty((rows, width // 2), dtype=gu.dtype, device=gu.device)
    _call("thn_clamped_glu", _ptr(out), _ptr(gu), rows, width // 2, float(limit), float(alpha), _code(gu, "clamped_glu"),
          _stream())
    return out


NORM_KINDS = {"rms": 1, "layer": 2, "as_is": 3}


@dataclass
class Gain:
    """A norm as the float32-residual kernels take it: ``weight`` float32 [width], ``offset`` 0
    for a gain stored as it multiplies and 1 for one stored around zero, ``eps``; ``kind`` "rms"
    (``x / sqrt(mean(x^2) + eps)``) or "layer" (``(x - mean) / sqrt(var + eps)``, with an optional
    ``bias`` float32 [width] added after the gain); "as_is" (as an output only): no norm, the
    stream itself rounded to the activation type."""

    weight: Optional[torch.Tensor]
    offset: float
    eps: float
    bias: Optional[torch.Tensor] = None
    kind: str = "rms"
    groups: int = 1     # "rms" as the norm of the stream: equal consecutive parts with statistics of their own


STREAM_AS_IS = Gain(None, 0.0, 1.0, None, "as_is")


def residual_norm(h: Optional[torch.Tensor], d: Optional[torch.Tensor], post: Optional[Gain], gain: Optional[Gain],
                  dtype: torch.dtype, d2: Optional[torch.Tensor] = None,
                  mult: float = 1.0) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """Norms around a residual stream ``h`` kept in float32 beside activations of ``dtype``:
    ``h <- h + mult * post(d + d2)`` in place (``post`` None: the branch is added as it is; ``d2``
    None: one branch; ``h`` None: the stream starts as that), then ``y = gain(h)`` of ``dtype``
    (``gain`` None: no y; ``STREAM_AS_IS``: y is h rounded).  See :class:`Gain` for the norms.
    Returns ``(h, y)``."""
    if d is None and h is None:
        raise KernelError("residual_norm: neither a stream nor a branch")
    h_is_new = h is None
    if d2 is not None:
        if d is None or tuple(d2.shape) != tuple(d.shape):
            raise KernelError("residual_norm: a second branch goes with a first of its shape")
        _need(d2, "residual_norm d2", dtype)
    if gain is not None and gain.groups != 1 and (gain.kind != "rms" or h is not None and h.shape[-1] % gain.groups):
        raise KernelError(f"residual_norm: {gain.groups} groups need an RMS norm over rows they divide")
    if post is not None and post.groups != 1:
        raise KernelError("residual_norm: the norm of a branch has no groups")
    if d is not None:
        _need(d, "residual_norm d", dtype)
    if h_is_new:
        h = torch.empty(d.shape, dtype=torch.float32, device=d.device)
    _need(h, "residual_norm h", torch.float32)
    if d is not None and tuple(d.shape) != tuple(h.shape):
        raise KernelError(f"residual_norm: shapes h {tuple(h.shape)}, d {tuple(d.shape)}")
    width = h.shape[-1]
    rows = h.numel() // width
    if post is not None and post.kind == "as_is":
        raise KernelError("residual_norm: 'as_is' is an output, not a norm of the branch")
    for g, what in ((post, "post"), (gain, "gain")):
        for t, name in (((g.weight, "gain"), (g.bias, "bias")) if g is not None else ()):
            if t is not None:
                _need(t, f"residual_norm {what} {name}", torch.float32)
                if t.shape[0] != width:
                    raise KernelError(f"residual_norm: {what} {name} has {t.shape[0]} entries, rows have {width}")
    y = torch.empty(h.shape, dtype=dtype, device=h.device) if gain is not None else None
    _call("thn_residual_norm", _ptr(y), _ptr(h), _ptr(d), _ptr(d2), float(mult), _ptr(post.weight) if post else None,
          _ptr(post.bias) if post else None, float(post.offset) if post else 0.0, float(post.eps) if post else 1.0,
          NORM_KINDS[post.kind] if post else 0, _ptr(gain.weight) if gain else None, _ptr(gain.bias) if gain else None,
          float(gain.offset) if gain else 0.0, float(gain.eps) if gain else 1.0, NORM_KINDS[gain.kind] if gain else 0,
          int(gain.groups) if gain else 1, rows, width, int(h_is_new), DTYPE_CODE[dtype], _stream())
    return h, y


GATE_KINDS = {"silu": 0, "logistic": 1}


def gated_head_norm(o: torch.Tensor, gate: torch.Tensor, gate_offset: int, weight: torch.Tensor, eps: float,
                    n_heads: int, size: int, dtype: torch.dtype, gate_kind: str = "silu", scale: float = 1.0,
                    out: Optional[torch.Tensor] = None, out_offset: int = 0) -> torch.Tensor:
    """o float32 [rows, heads, size] -> o / sqrt(mean over size + eps) * weight * act(gate), of
    ``dtype`` [rows, heads * size]; the gate of a row is ``gate[row, gate_offset : gate_offset +
    heads * size]``; ``weight`` has ``size`` entries (shared by the heads) or ``heads * size``;
    ``gate_kind`` "silu" or "logistic"; ``scale``: a constant factor on the result.  One head of
    ``heads * size`` entries is a norm over all heads together.  With ``out`` (rows of ``dtype``, at
    least ``out_offset + heads * size`` wide) the result goes to its columns from ``out_offset``."""
    _need(o, "gated_head_norm o", torch.float32)
    _need(gate, "gated_head_norm gate", dtype)
    _need(weight, "gated_head_norm weight", torch.float32)
    rows = o.shape[0]
    if o.numel() != rows * n_heads * size or weight.shape[0] not in (size, n_heads * size) or gate.shape[0] != rows \
            or gate_offset + n_heads * size > gate.shape[1]:
        raise KernelError(f"gated_head_norm: shapes o {tuple(o.shape)}, gate {tuple(gate.shape)}, weight {tuple(weight.shape)}")
    if out is None:
        out, out_offset = torch.empty((rows, n_heads * size), dtype=dtype, device=o.device), 0
    else:
        _need(out, "gated_head_norm out", dtype)
        if out.shape[0] != rows or out_offset < 0 or out_offset + n_heads * size > out.shape[1]:
            raise KernelError(f"gated_head_norm: out {tuple(out.shape)} has no room for {n_heads * size} columns from {out_offset}")
    gate_ptr = gate.data_ptr() + gate_offset * gate.element_size()
    _call("thn_gated_head_norm", out.data_ptr() + out_offset * out.element_size(), _ptr(o), gate_ptr, gate.shape[1],
          _ptr(weight), float(eps), rows, n_heads, size, int(weight.shape[0] != size and n_heads > 1), GATE_KINDS[gate_kind],
          out.shape[1], float(scale), DTYPE_CODE[dtype], _stream())
    return out


def rope_table(cos: torch.Tensor, sin: torch.Tensor, inv_freq: torch.Tensor, first: int, count: int) -> None:
    _need(cos, "rope_table cos", torch.float32)
    _need(sin, "rope_table sin", torch.float32)
    _need(inv_freq, "rope_table inv_freq", torch.float32)
    if first + count > cos.shape[0]:
        raise KernelError(f"rope_table: rows [{first}, {first + count}) exceed the table of {cos.shape[0]}")
    _call("thn_rope_table", _ptr(cos), _ptr(sin), _ptr(inv_freq), first, count, inv_freq.shape[0], _stream())


# ------------------------------------------------------------------ matrix products


def _sm_count_of(device) -> int:
    index = torch.device(device).index or 0
    if index not in _sm_count:
        _sm_count[index] = torch.cuda.get_device_properties(index).multi_processor_count
    return _sm_count[index]


# Products with at most STREAM_MAX_ROWS rows go to this library's weight-streaming kernel where it
# beats the vendor library (kernel_bench.py on B200, 1 to 16 rows, at the layer sizes of Qwen3-4B,
# -8B and -14B): a weight of at most STREAM_MAX_N rows (so few 128-row tiles that a cluster of
# four or more blocks shares each) under a reduction at least STREAM_MIN_K deep: o and down at
# 2560 x 4096, 2560 x 9728, 4096 x 4096, 4096 x 12288 (7.1 vs 10.3, 12.0 vs 20.4, 9.2 vs 12.2,
# 19.7 vs 31.3 us at 8 rows); and a weight of at least STREAM_MIN_N rows (the head: 123 vs 127,
# 191 vs 205, 233 vs 255 us).  The library wins on q/k/v and gate-up at every size (7.5 vs 10.0,
# 17.5 vs 21.0, 10.9 vs 13.2, 34.4 vs 36.8, 13.8 vs 16.7, 58.0 vs 59.5 us) and at 5120 x 5120 and
# 5120 x 17408 (11.5 vs 12.5, 31.2 vs 32.7 us).  The row limit comes from whole decode steps of
# the Qwen3-4B sizes, where a product also gains from starting under its predecessor's tail: with
# the streaming product a step of 17 / 24 / 32 / 33 / 48 / 64 rows takes 2.49 / 2.61 / 2.74 / 2.78 /
# 3.09 / 3.49 ms, with the library's 2.63 / 2.74 / 2.85 / 2.85 / 3.13 / 3.47 ms.
STREAM_MAX_ROWS = 48
STREAM_MIN_K = int(os.environ.get("THN_STREAM_MIN_K", 4096))
STREAM_MAX_N = int(os.environ.get("THN_STREAM_MAX_N", 4096))
STREAM_MIN_N = 65536
STREAM_POLICY = os.environ.get("THN_LINEAR_STREAM", "auto")     # auto | all | none (measurement)

_device_counters = {}


COUNTER_SLOTS = 1 << 20


def _counter_buffer(n: int, device) -> torch.Tensor:
    """Arrival counters for kernels whose last-arriving block finishes a shared result; zero
    between calls (the kernels reset them).  One buffer per device for the life of the
    process: captured graphs hold its address, so it is never replaced by a larger one."""
    if n > COUNTER_SLOTS:
        raise KernelError(f"a kernel asks for {n} arrival counters, the buffer holds {COUNTER_SLOTS}")
    index = torch.device(device).index or 0
    have = _device_counters.get(index)
    if have is None:
        have = torch.zeros(COUNTER_SLOTS, dtype=torch.int32, device=device)
        _device_counters[index] = have
    return have


_stream_needs = {}


def _stream_need(m: int, n: int, k: int, swiglu: bool, n_blocks: int):
    key = (m, n, k, swiglu, n_blocks)
    if key not in _stream_needs:
        floats, counters = ctypes.c_longlong(0), ctypes.c_int(0)
        lib().thn_gemm_stream_scratch(m, n, k, int(swiglu), n_blocks, ctypes.byref(floats), ctypes.byref(counters))
        _stream_needs[key] = (floats.value, counters.value)
    return _stream_needs[key]


def linear_stream(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16,
                  swiglu: bool = False, err: Optional[torch.Tensor] = None, n_blocks: int = 0) -> torch.Tensor:
    """The TMA / tcgen05 weight-streaming product for steps of at most 64 rows (bfloat16
    operands, K a multiple of 8) -> ``[M, N]`` in bfloat16 or float32.  With ``swiglu`` the
    weight is ``[2 * I, K]`` (gate rows, then up rows) and the result is ``silu(gate) * up``,
    ``[M, I]``, in one kernel.  ``n_blocks`` overrides how the work is cut (tests): that many
    blocks with balanced runs, or, negative, one thread-block cluster of that size per tile."""
    _need(x, "linear_stream x", torch.bfloat16)
    _need(weight, "linear_stream weight", torch.bfloat16)
    m, k = x.shape
    n = weight.shape[0] // 2 if swiglu else weight.shape[0]
    if weight.shape[1] != k or (swiglu and weight.shape[0] % 2):
        raise KernelError(f"linear_stream: shapes x {tuple(x.shape)}, weight {tuple(weight.shape)}")
    floats, n_counters = _stream_need(m, n, k, swiglu, n_blocks)
    counters = _counter_buffer(n_counters, x.device)
    scratch = torch.empty(floats, dtype=torch.float32, device=x.device)
    out = torch.empty((m, n), dtype=out_dtype, device=x.device)
    _call("thn_gemm_stream_bf16", _ptr(out), DTYPE_CODE[out_dtype], _ptr(scratch), _ptr(counters), _ptr(x),
          _ptr(weight), m, n, k, int(swiglu), n_blocks, _ptr(err), _stream())
    return out


def linear_tcgen05(x: torch.Tensor, weight: torch.Tensor, err: Optional[torch.Tensor] = None,
                   swiglu: bool = False) -> torch.Tensor:
    """The tcgen05 / TMEM / TMA product for steps with many rows: ``x [M, K] @ weight[N, K]^T``
    in bfloat16.  With ``swiglu`` the weight is ``[2 * I, K]`` (gate rows, then up rows) and the
    result is ``silu(gate) * up``, ``[M, I]``, in one kernel."""
    _need(x, "linear_tcgen05 x", torch.bfloat16)
    _need(weight, "linear_tcgen05 weight", torch.bfloat16)
    m, k = x.shape
    n = weight.shape[0] // 2 if swiglu else weight.shape[0]
    if weight.shape[1] != k:
        raise KernelError(f"linear_tcgen05: shapes x {tuple(x.shape)}, weight {tuple(weight.shape)}")
    out = torch.empty((m, n), dtype=torch.bfloat16, device=x.device)
    _call("thn_gemm_tcgen05_bf16", _ptr(out), _ptr(x), _ptr(weight), m, n, k, int(swiglu), _ptr(err), _stream())
    return out


def _stream_takes(m: int, n: int, k: int, fused: bool = False) -> bool:
    if STREAM_POLICY == "none" or not lib().thn_gemm_stream_supported(m, n, k):
        return False
    if STREAM_POLICY == "all":
        return True
    return not fused and m <= STREAM_MAX_ROWS and ((k >= STREAM_MIN_K and n <= STREAM_MAX_N) or n >= STREAM_MIN_N)


def linear_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor, err: Optional[torch.Tensor] = None) -> torch.Tensor:
    """silu(x gate^T) * (x up^T) for ``w_gate_up = cat(gate, up)``: one kernel where the
    weight-streaming product takes the shape, else the product followed by the activation."""
    if x.dtype == torch.bfloat16 and _stream_takes(x.shape[0], w_gate_up.shape[0] // 2, x.shape[1], fused=True):
        return linear_stream(x, w_gate_up, swiglu=True, err=err)
    return swiglu(linear(x, w_gate_up, err=err))


def linear(x: torch.Tensor, weight: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
           err: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [M, K] @ weight[N, K]^T.  float32: this library's FFMA kernel.  bfloat16 with few
    rows and a deep reduction or a tall weight: this library's weight-streaming kernel
    (``err``: the step's device error word for its bounded waits).  bfloat16 with a float32 result
    of at most 64 columns (a router, a gate): this library's warp-per-row kernel.  bfloat16 otherwise: the
    vendor library's tensor-core product with float32 accumulation (the reference's choice,
    engine/engine.py:341-350).  ``out_dtype=torch.float32`` keeps the accumulator's
    precision (used for logits).  ``bias`` (of the activation type, ``[N]``) is added to every row:
    in the vendor product's epilogue (float32, before the one rounding), or by a kernel of its own
    after the FFMA product."""
    if bias is not None:
        _need(bias, "linear bias", x.dtype)
        if bias.shape[0] != weight.shape[0]:
            raise KernelError(f"linear: a bias of {bias.shape[0]} entries for {weight.shape[0]} outputs")
        if x.dtype == torch.float32:
            out = linear(x, weight, out_dtype, err)
            _call("thn_add_bias_f32", _ptr(out), _ptr(bias), out.shape[0], out.shape[1], 1.0, _stream())
            return out
        _need(x, "linear x")
        _need(weight, "linear weight", x.dtype)
        if out_dtype in (None, torch.bfloat16):
            return torch.nn.functional.linear(x, weight, bias)
        out = torch.mm(x, weight.t(), out_dtype=out_dtype)
        _call("thn_add_bias_f32", _ptr(out), _ptr(bias.float()), out.shape[0], out.shape[1], 1.0, _stream())
        return out
    _need(x, "linear x")
    _need(weight, "linear weight", x.dtype)
    if x.dim() != 2 or weight.dim() != 2 or x.shape[1] != weight.shape[1]:
        raise KernelError(f"linear: shapes x {tuple(x.shape)}, weight {tuple(weight.shape)}")
    if x.dtype == torch.float32:
        out = torch.empty((x.shape[0], weight.shape[0]), dtype=torch.float32, device=x.device)
        _call("thn_gemm_f32", _ptr(out), _ptr(x), _ptr(weight), x.shape[0], weight.shape[0], x.shape[1], _stream())
        return out
    if x.dtype != torch.bfloat16:
        raise KernelError(f"linear: dtype {x.dtype} is not supported")
    if (out_dtype == torch.float32 and lib().thn_linear_skinny_supported(weight.shape[0], x.shape[1])
            and (x.data_ptr() | weight.data_ptr()) % 16 == 0):
        # a router or a gate: a few float32 outputs per row, on this library's warp-per-row kernel
        out = torch.empty((x.shape[0], weight.shape[0]), dtype=torch.float32, device=x.device)
        _call("thn_linear_skinny_bf16", _ptr(out), _ptr(x), _ptr(weight), x.shape[0], weight.shape[0], x.shape[1], _stream())
        return out
    if _stream_takes(x.shape[0], weight.shape[0], x.shape[1]):
        return linear_stream(x, weight, out_dtype or torch.bfloat16, err=err)
    if out_dtype in (None, torch.bfloat16):
        return torch.nn.functional.linear(x, weight)
    return torch.mm(x, weight.t(), out_dtype=out_dtype)


# ------------------------------------------------------------------ attention


@dataclass
class KVView:
    """One cache entry as the kernels see it."""

    storage: torch.Tensor       # [pages, 2, n_kv, page_size, head_dim] of this entry
    block_table: torch.Tensor   # int32 [max_slots, max_pages_per_seq]
    n_kv: int
    page_size: int
    head_dim: int
    value_dim: Optional[int] = None   # size of a value where it differs from a key's (storage is then
                                      # [pages, n_kv * page_size * (head_dim + value_dim)], K block then V block)

    @property
    def v_dim(self) -> int:
        return self.head_dim if self.value_dim is None else self.value_dim


@dataclass(frozen=True)
class ScoreShape:
    """What happens to an attention score between the scale and the softmax.  ``temp_every`` > 0:
    the scores of the query at position p are multiplied by
    ``1 + temp_coef * ln(floor((p + 1) / temp_every) + 1)``.  ``softcap`` > 0: a score s becomes
    ``softcap * tanh(s / softcap)``.  In this order; zeros: neither."""

    softcap: float = 0.0
    temp_coef: float = 0.0
    temp_every: int = 0

    @property
    def active(self) -> bool:
        return self.softcap > 0.0 or self.temp_every > 0

    def args(self):
        return float(self.softcap), float(self.temp_coef), int(self.temp_every)


PLAIN_SCORES = ScoreShape()


@dataclass
class RowTiles:
    """Tiles of at most ``size`` consecutive rows of one sequence, for the prompt attention
    kernels: first packed row and row count of each tile (int32, on the device).  The
    kernels start at the end of the list, so it is ordered by the keys a tile sees,
    fewest first (see :func:`row_tiles_of`)."""

    row0: torch.Tensor
    rows: torch.Tensor
    n: int
    size: int


def row_tiles_of(counts, held, size: int):
    """Host lists (row0, rows) of the tiles of a step whose sequences bring ``counts[i]``
    rows on top of ``held[i]`` cached tokens, fewest keys first."""
    tiles, start = [], 0
    for c, h in zip(counts, held):
        for r in range(0, c, size):
            n = min(size, c - r)
            tiles.append((h + r + n, start + r, n))
        start += c
    tiles.sort()
    return [t[1] for t in tiles], [t[2] for t in tiles]


@dataclass
class RotaryTables:
    cos: torch.Tensor   # float32 [positions, rotary_dim / 2]
    sin: torch.Tensor
    rotary_dim: int
    layout: str = "half"    # which entries make a pair: "half" (i, i + rotary_dim / 2) or "interleaved" (2i, 2i + 1)


def qk_norm_rope_cache(qkv, q_gain: Optional[torch.Tensor], k_gain: Optional[torch.Tensor],
                       eps: float, rotary: Optional[RotaryTables], rows: StepRows, kv: KVView, n_q: int,
                       write_cache: bool, err: torch.Tensor) -> torch.Tensor:
    """qkv -> q, normalised and rotated; K and V go to the cache."""
    width = (n_q + 2 * kv.n_kv) * kv.head_dim
    if tuple(qkv.shape) != (rows.n_rows, width):
        raise KernelError(f"qk_norm_rope_cache: qkv is {tuple(qkv.shape)}, expected {(rows.n_rows, width)}")
    if kv.storage.dtype != qkv.dtype:
        raise KernelError(f"qk_norm_rope_cache: cache is {kv.storage.dtype}, activations {qkv.dtype}")
    _need(qkv, "qk_norm_rope_cache qkv")
    q = torch.empty((rows.n_rows, n_q * kv.head_dim), dtype=qkv.dtype, device=kv.storage.device)
    w_code = _code(q_gain, "qk gains") if q_gain is not None else DTYPE_CODE[qkv.dtype]
    _call("thn_qk_norm_rope_cache", _ptr(q), _ptr(qkv), _ptr(q_gain), _ptr(k_gain), w_code, float(eps),
          _ptr(rotary.cos) if rotary else None, _ptr(rotary.sin) if rotary else None,
          rotary.cos.shape[0] if rotary else 0, rotary.rotary_dim if rotary else 0,
          _ptr(rows.row_slot), _ptr(rows.row_pos), _ptr(kv.storage), _ptr(kv.block_table),
          kv.block_table.shape[1], kv.n_kv, kv.page_size, kv.head_dim, rows.n_rows, n_q, int(write_cache),
          DTYPE_CODE[qkv.dtype], _ptr(err), _stream())
    return q


def attention_generic(q: torch.Tensor, rows: StepRows, kv: KVView, n_q: int, scale: float,
                      window: Optional[int], err: torch.Tensor, keep_first: int = 0, chunk: Optional[int] = None,
                      exact_weights: bool = False, shape: ScoreShape = PLAIN_SCORES,
                      sinks: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One warp per (row, head), any sizes.  ``chunk``: a row sees only the keys of its own chunk
    of that many positions; ``exact_weights``: the softmax weights stay float32 where they
    multiply the values; the output has ``kv.v_dim`` entries per head.  ``sinks`` (float32
    ``[n_q]``): the softmax's denominator of head h also holds ``exp(sinks[h])``, a term without
    key and value."""
    _need(q, "attention q")
    if sinks is not None:
        _need(sinks, "attention sinks", torch.float32)
        if sinks.shape[0] != n_q:
            raise KernelError(f"attention: {sinks.shape[0]} sinks for {n_q} heads")
    out = torch.empty((q.shape[0], n_q * kv.v_dim), dtype=q.dtype, device=q.device)
    _call("thn_attention_generic", _ptr(out), _ptr(q), _ptr(rows.row_slot), _ptr(rows.row_pos), _ptr(kv.storage),
          _ptr(kv.block_table), kv.block_table.shape[1], kv.n_kv, kv.page_size, kv.head_dim, kv.v_dim, rows.n_rows, n_q,
          float(scale), int(window or 0), int(keep_first or 0), int(chunk or 0), int(bool(exact_weights)), *shape.args(),
          _ptr(sinks), _code(q, "attention"), _ptr(err), _stream())
    return out


QK_NORM_SCOPES = {None: 0, "none": 0, "head": 1, "projection": 2}
ROTARY_LAYOUTS = {"half": 0, "interleaved": 1}


def qk_prepare(proj: torch.Tensor, q_gain: Optional[torch.Tensor], k_gain: Optional[torch.Tensor], norm_scope: str,
               eps: float, rotary: Optional[RotaryTables], rows: StepRows, kv: KVView, n_q: int,
               values_are_keys: bool, write_cache: bool, err: torch.Tensor, gain_offset: float = 0.0,
               value_rotary: Optional[RotaryTables] = None, proj_offset: int = 0) -> torch.Tensor:
    """From projected rows ``[q | k | v]`` (or ``[q | k]`` when the values are the keys as
    projected) to queries; keys and values go to the cache.  ``norm_scope``: "head" (an RMS norm
    per head, gains ``[head_dim]``), "projection" (one RMS norm over all heads of q and one over
    all heads of k, gains of those sizes) or None; the rotation follows ``rotary.layout``.
    Float32 inside, one rounding at the store.  ``value_rotary``: tables by which the values are
    turned (their first ``rotary_dim`` entries, the keys' layout of pairs) before they go to the
    cache.  ``proj_offset``: the column of ``proj`` at which ``[q | k | v]`` starts (a slice of a
    wider projected row)."""
    if value_rotary is not None and rotary is not None and value_rotary.layout != rotary.layout:
        raise KernelError("qk_prepare: keys and values turn in one layout of pairs")
    layout = rotary.layout if rotary else (value_rotary.layout if value_rotary else "half")
    _need(proj, "qk_prepare proj")
    if kv.storage.dtype != proj.dtype:
        raise KernelError(f"qk_prepare: cache is {kv.storage.dtype}, activations {proj.dtype}")
    if proj.shape[0] != rows.n_rows:
        raise KernelError(f"qk_prepare: {proj.shape[0]} projected rows for a step of {rows.n_rows}")
    scope = QK_NORM_SCOPES[norm_scope]
    if scope:
        want_q, want_k = (kv.head_dim, kv.head_dim) if scope == 1 else (n_q * kv.head_dim, kv.n_kv * kv.head_dim)
        _need(q_gain, "qk_prepare q gain", torch.float32)
        _need(k_gain, "qk_prepare k gain", torch.float32)
        if q_gain.shape[0] != want_q or k_gain.shape[0] != want_k:
            raise KernelError(f"qk_prepare: gains of {q_gain.shape[0]} and {k_gain.shape[0]} entries, expected "
                              f"{want_q} and {want_k}")
    q = torch.empty((rows.n_rows, n_q * kv.head_dim), dtype=proj.dtype, device=proj.device)
    if values_are_keys and kv.v_dim != kv.head_dim:
        raise KernelError("qk_prepare: values that are the keys have the keys' size")
    if proj_offset < 0 or proj_offset + (n_q + kv.n_kv) * kv.head_dim + (0 if values_are_keys else kv.n_kv * kv.v_dim) > proj.shape[1]:
        raise KernelError(f"qk_prepare: rows of {proj.shape[1]} hold no q, k, v from column {proj_offset}")
    _call("thn_qk_prepare", _ptr(q), proj.data_ptr() + proj_offset * proj.element_size(), proj.shape[1],
          _ptr(q_gain) if scope else None,
          _ptr(k_gain) if scope else None, scope, float(gain_offset), float(eps),
          _ptr(rotary.cos) if rotary else None, _ptr(rotary.sin) if rotary else None,
          rotary.cos.shape[0] if rotary else 0, rotary.rotary_dim if rotary else 0,
          ROTARY_LAYOUTS[layout], int(bool(values_are_keys)), _ptr(rows.row_slot),
          _ptr(rows.row_pos), _ptr(kv.storage), _ptr(kv.block_table), kv.block_table.shape[1], kv.n_kv, kv.page_size,
          kv.head_dim, kv.v_dim, rows.n_rows, n_q, int(bool(write_cache)),
          _ptr(value_rotary.cos) if value_rotary else None, _ptr(value_rotary.sin) if value_rotary else None,
          value_rotary.cos.shape[0] if value_rotary else 0, value_rotary.rotary_dim if value_rotary else 0,
          DTYPE_CODE[proj.dtype], _ptr(err), _stream())
    return q


def prompt_attention_tile(dtype: torch.dtype, kv_head_dim: int, page_size: int, n_q: int, n_kv: int,
                          value_dim: Optional[int] = None, chunk: Optional[int] = None) -> int:
    """Rows per tile that the prompt attention kernel for these sizes works on, or 0 if the
    sizes go to the kernel that needs no tiles."""
    if value_dim is not None and value_dim != kv_head_dim:
        return 0
    if dtype == torch.bfloat16 and lib().thn_attention_mma_supported(kv_head_dim, page_size, n_q, n_kv):
        return lib().thn_attention_prefill_tile_rows()
    return 0


def attention(q: torch.Tensor, rows: StepRows, kv: KVView, n_q: int, scale: float, window: Optional[int],
              err: torch.Tensor, tiles: Optional[RowTiles] = None, keep_first: int = 0,
              chunk: Optional[int] = None, exact_weights: bool = False,
              shape: ScoreShape = PLAIN_SCORES, sinks: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal attention of the step's rows over the cache (which already holds the step's
    own keys).  Chooses the kernel by dtype, head size and step shape; the tensor-core
    kernels for steps of several tokens per sequence need ``tiles``.  With a window,
    ``keep_first`` keys at the start of a sequence stay visible to every later row.  With
    ``chunk`` a row sees the keys of its own chunk of that many positions only.
    ``exact_weights`` asks for softmax weights that are not rounded to bfloat16 in the product
    with the values: float32 in the kernel without tensor cores, two bfloat16 parts (the weight's
    rounding and what the rounding left) in the ``mma.sync`` kernels.  The tcgen05 prompt kernel
    (head size 128) has one bfloat16 part only and is taken all the same: it is 2.4 to 3.6 times
    faster there than the ``mma.sync`` kernel with two parts; ``THN_ATTN_TCGEN05=0`` sends those
    prompts to the latter.  ``shape``: a position-dependent factor on a row's scores and a tanh
    cap (:class:`ScoreShape`), taken by every kernel but the streaming decode kernel.  ``sinks``: a
    term ``exp(sinks[h])`` without key and value in the softmax's denominator of head h; the
    warp-per-(row, head) kernel, the ``mma.sync`` kernels and the tcgen05 prompt kernel take it (the
    streaming decode kernel does not, and is not chosen then)."""
    keep_first = int(keep_first or 0) if window else 0
    if kv.v_dim != kv.head_dim:
        return attention_generic(q, rows, kv, n_q, scale, window, err, keep_first, chunk, exact_weights, shape, sinks)
    if q.dtype == torch.bfloat16 and lib().thn_attention_mma_supported(kv.head_dim, kv.page_size, n_q, kv.n_kv):
        if rows.max_q_len == 1:
            return attention_decode_bf16(q, rows, kv, n_q, scale, window, err, keep_first=keep_first, chunk=chunk,
                                         split_weights=exact_weights, shape=shape, sinks=sinks)
        if tiles is not None:
            if USE_TCGEN05_ATTENTION and lib().thn_attention_tcgen05_supported(kv.head_dim, kv.page_size, n_q, kv.n_kv):
                return attention_prefill_tcgen05(q, rows, tiles, kv, n_q, scale, window, err, keep_first, chunk, shape, sinks)
            return attention_prefill_bf16(q, rows, tiles, kv, n_q, scale, window, err, keep_first, chunk, exact_weights,
                                          shape, sinks)
    return attention_generic(q, rows, kv, n_q, scale, window, err, keep_first, chunk, exact_weights, shape, sinks)


def attention_prefill_tcgen05(q: torch.Tensor, rows: StepRows, tiles: RowTiles, kv: KVView, n_q: int, scale: float,
                              window: Optional[int], err: torch.Tensor, keep_first: int = 0,
                              chunk: Optional[int] = None, shape: ScoreShape = PLAIN_SCORES,
                              sinks: Optional[torch.Tensor] = None) -> torch.Tensor:
    """tcgen05 / TMEM / TMA flash attention for steps with several tokens per sequence
    (bfloat16, head size 128)."""
    _need(q, "attention q", torch.bfloat16)
    out = torch.empty_like(q)
    _check_tiles(tiles)
    _call("thn_attention_prefill_tcgen05", _ptr(out), _ptr(q), _ptr(tiles.row0), _ptr(tiles.rows),
          tiles.n, q.shape[0], _ptr(rows.row_slot), _ptr(rows.row_pos), _ptr(kv.storage), kv.storage.shape[0],
          _ptr(kv.block_table), kv.block_table.shape[1], kv.n_kv, kv.page_size, kv.head_dim, n_q, float(scale),
          int(window or 0), int(keep_first or 0), int(chunk or 0), *shape.args(), _ptr(sinks), _ptr(err), _stream())
    return out


USE_TCGEN05_ATTENTION = os.environ.get("THN_ATTN_TCGEN05", "1").strip().lower() not in ("0", "false", "no", "off")


def ROW_TILE() -> int:
    """Rows per tile that the tensor-core prompt attention kernels work on."""
    return lib().thn_attention_prefill_tile_rows()


def _check_tiles(tiles: RowTiles) -> None:
    if tiles.size != ROW_TILE():
        raise KernelError(f"prompt attention: row tiles of {tiles.size} rows, the kernel works on {ROW_TILE()}")
    _need(tiles.row0, "row tiles", torch.int32)
    _need(tiles.rows, "row tiles", torch.int32)


def attention_prefill_bf16(q: torch.Tensor, rows: StepRows, tiles: RowTiles, kv: KVView, n_q: int, scale: float,
                           window: Optional[int], err: torch.Tensor, keep_first: int = 0,
                           chunk: Optional[int] = None, split_weights: bool = False,
                           shape: ScoreShape = PLAIN_SCORES, sinks: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Tensor-core flash attention for steps with several tokens per sequence.  ``split_weights``:
    the softmax weights multiply the values as two bfloat16 parts (two products), not one."""
    _need(q, "attention q", torch.bfloat16)
    out = torch.empty_like(q)
    _check_tiles(tiles)
    _call("thn_attention_prefill_bf16", _ptr(out), _ptr(q), _ptr(tiles.row0), _ptr(tiles.rows),
          tiles.n, _ptr(rows.row_slot), _ptr(rows.row_pos), _ptr(kv.storage), _ptr(kv.block_table),
          kv.block_table.shape[1], kv.n_kv, kv.page_size, kv.head_dim, n_q, float(scale), int(window or 0),
          int(keep_first or 0), int(chunk or 0), int(bool(split_weights)), *shape.args(), _ptr(sinks), _ptr(err), _stream())
    return out


DECODE_MAX_SPLITS = 32     # the splits of a key range are combined by the lanes of one warp


def decode_splits(n_seqs: int, n_kv: int, device, head_dim: int = 128, fused: bool = False,
                  context: Optional[int] = None, differ: Optional[bool] = None) -> int:
    """Splits of the key range per (sequence, kv head) of a single-token step: as many as fill
    the SMs once, the splits of a pair being the blocks of one thread-block cluster (at most
    eight, six unless the pairs are very few), all clusters resident at once.  It depends on the
    batch and on ``context`` (the step's ``max_context``, a bound that holds for every replay of
    a captured step), never on the lengths themselves."""
    if os.environ.get("THN_DECODE_SPLITS"):
        return int(os.environ["THN_DECODE_SPLITS"])
    pairs = max(1, n_seqs * n_kv)
    if long_sequences_stream(n_seqs, n_kv, context, differ, device):
        return 1           # unsplit: the streaming kernel's step
    one_wave = lib().thn_attention_decode_one_wave_splits(head_dim, int(fused), pairs)
    if context is not None and context >= LONG_CONTEXT:
        # Few long sequences: a block works through its tiles one after the other, and a cluster's
        # blocks are too few to draw the memory bandwidth.  Two blocks per SM, meeting in global
        # memory, read 32,768 keys of one sequence in 33 us against 56 us (B200, 8 kv heads);
        # below 8,192 keys the cluster's cheaper merge wins.
        wide = min(DECODE_MAX_SPLITS, 2 * _sm_count_of(device) // pairs)
        if wide >= 2 * max(1, one_wave):
            return wide
    return max(1, one_wave)


def long_sequences_stream(n_seqs: int, n_kv: int, context: Optional[int], differ: Optional[bool], device) -> bool:
    """Whether a single-token step is one for the streaming decode attention by what the host
    knows: sequences that may hold STREAM_MIN_CONTEXT keys or more, about as many (sequence, kv
    head) pairs as SMs or more, and, if the lengths differ, at least two pairs per resident
    block, so that long and short ones can be paired (with one pair per block the longest
    sequence alone would set the time: 4.18 against 4.08 ms per step at batch 16 with 117 to
    2,026 keys, Qwen3-8B sizes).  Measured on B200, Qwen3-4B sizes, equal lengths, ms per step
    with one block or one cluster per pair against the streaming kernel: batch 16 / 24 / 32 / 48
    at 2,048 keys 3.03 / 3.51 / 3.87 / 4.90 against 2.98 / 3.36 / 3.78 / 4.64; at 4,096 keys
    3.85 / 4.76 / 5.42 / 7.46 against 3.69 / 4.38 / 5.18 / 6.75; level at 1,024 keys; batch 12
    and below: the cluster."""
    if context is None or context < STREAM_MIN_CONTEXT or not lib().thn_attention_decode_streams():
        return False
    pairs, sms = n_seqs * n_kv, _sm_count_of(device)
    if differ is not False:
        return pairs >= 4 * sms          # two blocks per SM, two pairs per block
    return pairs * 20 >= 17 * sms


def decode_hints(rows: StepRows, n_kv: int, n_splits: int, device) -> int:
    """What the host knows of a single-token step, as the kernels' ``hints`` bits: 1 unless the
    sequences are known to be about equally long; 2 if the step is unsplit and
    :func:`long_sequences_stream` says so."""
    hints = 0 if rows.lengths_differ is False else 1
    if n_splits == 1 and long_sequences_stream(rows.n_rows, n_kv, rows.max_context, rows.lengths_differ, device):
        hints |= 2
    return hints


def attention_decode_bf16(q: torch.Tensor, rows: StepRows, kv: KVView, n_q: int, scale: float,
                          window: Optional[int], err: torch.Tensor, n_splits: Optional[int] = None,
                          scratch: Optional[torch.Tensor] = None, fused_merge: bool = True,
                          keep_first: int = 0, chunk: Optional[int] = None, split_weights: bool = False,
                          shape: ScoreShape = PLAIN_SCORES, sinks: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Split-KV flash decoding: one token per sequence.  Partial results of the splits go
    through float32 scratch memory, which is allocated here unless given."""
    _need(q, "attention q", torch.bfloat16)
    n_seqs = rows.n_rows
    if n_splits is None:
        n_splits = decode_splits(n_seqs, kv.n_kv, q.device, kv.head_dim, context=rows.max_context,
                                 differ=rows.lengths_differ)
    need = lib().thn_attention_decode_scratch_floats(n_seqs, n_q, n_splits, kv.head_dim)
    if need and scratch is None:
        scratch = torch.empty(need, dtype=torch.float32, device=q.device)
    if need and scratch.numel() < need:
        raise KernelError(f"attention_decode: scratch has {scratch.numel()} floats, {need} needed")
    counters = _counter_buffer(n_seqs * kv.n_kv, q.device) if n_splits > 1 and fused_merge else None
    out = torch.empty_like(q)
    _call("thn_attention_decode_bf16", _ptr(out), _ptr(q), _ptr(rows.row_slot), _ptr(rows.row_pos),
          _ptr(kv.storage), _ptr(kv.block_table), kv.block_table.shape[1], kv.n_kv, kv.page_size, kv.head_dim,
          n_seqs, n_q, n_splits, float(scale), int(window or 0), int(keep_first or 0), int(chunk or 0),
          int(bool(split_weights)), *shape.args(), _ptr(sinks), _ptr(scratch), _ptr(counters),
          kv.storage.shape[0], decode_hints(rows, kv.n_kv, n_splits, q.device), _ptr(err), _stream())
    return out


FUSE_DECODE_ATTENTION = os.environ.get("THN_FUSE_DECODE", "1").strip().lower() not in ("0", "false", "no", "off")


def qkv_attention(qkv: torch.Tensor, q_gain: Optional[torch.Tensor], k_gain: Optional[torch.Tensor], eps: float,
                  rotary: Optional[RotaryTables], rows: StepRows, kv: KVView, n_q: int, scale: float,
                  window: Optional[int], write_cache: bool, err: torch.Tensor,
                  tiles: Optional[RowTiles] = None) -> torch.Tensor:
    """From the raw q/k/v rows of a step to the attention output: per-head q/k norm, rotation,
    cache write and attention over the cache.  One kernel for single-token steps in bfloat16
    with head norm and full rotation at the tensor-core kernel's sizes; otherwise
    :func:`qk_norm_rope_cache` followed by :func:`attention`."""
    fusable = (FUSE_DECODE_ATTENTION and rows.max_q_len == 1
               and qkv.dtype == torch.bfloat16 and q_gain is not None and k_gain is not None and rotary is not None
               and rotary.rotary_dim == kv.head_dim and kv.storage.dtype == torch.bfloat16
               and lib().thn_attention_fused_supported(kv.head_dim, kv.page_size, n_q, kv.n_kv))
    if not fusable:
        q = qk_norm_rope_cache(qkv, q_gain, k_gain, eps, rotary, rows, kv, n_q, write_cache, err)
        return attention(q, rows, kv, n_q, scale, window, err, tiles)
    n_seqs = rows.n_rows
    width = (n_q + 2 * kv.n_kv) * kv.head_dim
    if tuple(qkv.shape) != (n_seqs, width):
        raise KernelError(f"qkv_attention: qkv is {tuple(qkv.shape)}, expected {(n_seqs, width)}")
    n_splits = decode_splits(n_seqs, kv.n_kv, qkv.device, kv.head_dim, fused=True, context=rows.max_context,
                             differ=rows.lengths_differ)
    need = lib().thn_attention_decode_scratch_floats(n_seqs, n_q, n_splits, kv.head_dim)
    scratch = torch.empty(need, dtype=torch.float32, device=qkv.device) if need else None
    counters = _counter_buffer(n_seqs * kv.n_kv, qkv.device) if n_splits > 1 else None
    out = torch.empty((n_seqs, n_q * kv.head_dim), dtype=torch.bfloat16, device=qkv.device)
    _call("thn_attention_decode_fused_bf16", _ptr(out), _ptr(qkv), _ptr(q_gain), _ptr(k_gain),
          _code(q_gain, "qk gains"), float(eps), _ptr(rotary.cos), _ptr(rotary.sin), rotary.cos.shape[0],
          int(bool(write_cache)), _ptr(rows.row_slot), _ptr(rows.row_pos), _ptr(kv.storage), _ptr(kv.block_table),
          kv.block_table.shape[1], kv.n_kv, kv.page_size, kv.head_dim, n_seqs, n_q, n_splits, float(scale),
          int(window or 0), _ptr(scratch), _ptr(counters), kv.storage.shape[0],
          decode_hints(rows, kv.n_kv, n_splits, qkv.device), _ptr(err), _stream())
    return out


# ------------------------------------------------------------------ gated delta rule


@dataclass
class DeltaShape:
    """Sizes of a gated-delta-rule mixer.  A projected row holds, in this order, the columns
    q and k (``n_kv * key_dim`` each), v and the output gate (``n_heads * value_dim`` each), the
    write strength and the decay input (``n_heads`` each)."""

    n_heads: int
    n_kv: int
    key_dim: int
    value_dim: int
    taps: int

    @property
    def conv_channels(self) -> int:
        return 2 * self.n_kv * self.key_dim + self.n_heads * self.value_dim

    @property
    def gate_offset(self) -> int:
        return self.conv_channels

    @property
    def proj_width(self) -> int:
        return self.conv_channels + self.n_heads * self.value_dim + 2 * self.n_heads


def _delta_check(proj: torch.Tensor, conv_w: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor,
                 state: torch.Tensor, ring: torch.Tensor, shape: DeltaShape, what: str) -> None:
    _need(proj, f"{what} proj")
    _need(conv_w, f"{what} conv_w", torch.float32)
    _need(a_log, f"{what} a_log", torch.float32)
    _need(dt_bias, f"{what} dt_bias", torch.float32)
    _need(state, f"{what} state", torch.float32)
    _need(ring, f"{what} ring", proj.dtype)
    if proj.shape[1] != shape.proj_width or tuple(conv_w.shape) != (shape.conv_channels, shape.taps) \
            or a_log.shape[0] != shape.n_heads or dt_bias.shape[0] != shape.n_heads \
            or tuple(state.shape[1:]) != (shape.n_heads, shape.value_dim, shape.key_dim) \
            or tuple(ring.shape[1:]) != (shape.taps, shape.conv_channels) or ring.shape[0] != state.shape[0]:
        raise KernelError(f"{what}: shapes proj {tuple(proj.shape)}, conv_w {tuple(conv_w.shape)}, state "
                          f"{tuple(state.shape)}, ring {tuple(ring.shape)} do not fit {shape}")


DELTA_LANES = int(os.environ.get("THN_DELTA_LANES", 0))     # 8 or 32 lanes per state column; 0: by the step's size
FUSE_DELTA_DECODE = os.environ.get("THN_FUSE_DELTA_DECODE", "1").strip().lower() not in ("0", "false", "no", "off")


def delta_rule(proj: torch.Tensor, conv_w: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor,
               state: torch.Tensor, ring: torch.Tensor, rows: StepRows, seq_lens: torch.Tensor, shape: DeltaShape,
               unit_eps: float) -> torch.Tensor:
    """The gated delta rule over a step's rows: short causal convolutions of q, k and v with
    silu, unit norms of q (also scaled by ``key_dim ** -0.5``) and k, write strength and decay,
    and per head ``S <- g S; u = b (v - S^T k); S <- S + k u^T; o = S^T q`` from the state the
    sequences' earlier steps left.  ``state`` float32 [slots, heads, value_dim, key_dim] and
    ``ring`` [slots, taps, channels] (the raw projection of position p at p mod taps) are read
    and updated; ``seq_lens`` holds the tokens each slot held before the step.  Returns the
    read-out, float32 [rows, heads, value_dim].  Steps of one token per sequence run as one
    kernel; others as three (prepare, recurrence, ring update).  With float32 activations the
    recurrence carries the state in double between a step's first and last token."""
    _delta_check(proj, conv_w, a_log, dt_bias, state, ring, shape, "delta_rule")
    if proj.shape[0] != rows.n_rows:
        raise KernelError(f"delta_rule: {proj.shape[0]} projected rows for a step of {rows.n_rows}")
    n, dev = rows.n_rows, proj.device
    s = shape
    o = torch.empty((n, s.n_heads, s.value_dim), dtype=torch.float32, device=dev)
    code = DTYPE_CODE[proj.dtype]
    if rows.max_q_len == 1 and FUSE_DELTA_DECODE:
        _call("thn_delta_decode", _ptr(o), _ptr(state), _ptr(ring), _ptr(proj), _ptr(conv_w), _ptr(a_log), _ptr(dt_bias),
              _ptr(rows.row_slot), _ptr(rows.row_pos), n, s.n_heads, s.n_kv, s.key_dim, s.value_dim, s.taps,
              s.proj_width, float(unit_eps), code, _stream())
        return o
    qn = torch.empty((n, s.n_kv, s.key_dim), dtype=torch.float32, device=dev)
    kn = torch.empty_like(qn)
    vc = torch.empty((n, s.n_heads, s.value_dim), dtype=torch.float32, device=dev)
    beta = torch.empty((n, s.n_heads), dtype=torch.float32, device=dev)
    decay = torch.empty_like(beta)
    _call("thn_delta_prepare", _ptr(qn), _ptr(kn), _ptr(vc), _ptr(beta), _ptr(decay), _ptr(proj), _ptr(conv_w),
          _ptr(a_log), _ptr(dt_bias), _ptr(ring), _ptr(rows.row_slot), _ptr(rows.row_pos), _ptr(seq_lens), n,
          s.n_heads, s.n_kv, s.key_dim, s.value_dim, s.taps, s.proj_width, float(unit_eps), code, _stream())
    _call("thn_delta_recurrence", _ptr(o), _ptr(state), _ptr(qn), _ptr(kn), _ptr(vc), _ptr(beta), _ptr(decay),
          _ptr(rows.cu_seqlens), _ptr(rows.slots), rows.n_seqs, s.n_heads, s.n_kv, s.key_dim, s.value_dim,
          int(proj.dtype == torch.float32), DELTA_LANES, _stream())
    _call("thn_delta_conv_ring_update", _ptr(ring), _ptr(proj), _ptr(rows.cu_seqlens), _ptr(rows.slots), _ptr(seq_lens),
          rows.n_seqs, s.n_heads, s.n_kv, s.key_dim, s.value_dim, s.taps, s.proj_width, code, _stream())
    return o


# ------------------------------------------------------------------ latent attention


def latent_norm(proj: torch.Tensor, offset: int, rank: int, gain: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm of the ``rank`` entries from column ``offset`` of every projected row, times
    ``gain`` (float32 [rank]) -> [rows, rank] of the rows' type: the latent that the
    up-projection reads."""
    _need(proj, "latent_norm proj")
    _need(gain, "latent_norm gain", torch.float32)
    if gain.shape[0] != rank or offset + rank > proj.shape[1]:
        raise KernelError(f"latent_norm: {rank} entries from column {offset} of rows of {proj.shape[1]}, gain {tuple(gain.shape)}")
    out = torch.empty((proj.shape[0], rank), dtype=proj.dtype, device=proj.device)
    _call("thn_latent_norm", _ptr(out), proj.data_ptr() + offset * proj.element_size(), proj.shape[1], _ptr(gain),
          float(eps), proj.shape[0], rank, _code(proj, "latent_norm"), _stream())
    return out


def latent_assemble(proj: torch.Tensor, q_offset: int, shared_offset: int, up: torch.Tensor,
                    rotary: Optional[RotaryTables], rows: StepRows, kv: KVView, n_heads: int, plain: int, rot: int,
                    err: torch.Tensor, value_dim: Optional[int] = None) -> torch.Tensor:
    """Queries and cache entries of latent attention.  ``proj`` rows hold the queries
    ``[heads][plain | rot]`` from column ``q_offset`` and one shared key part of ``rot`` entries
    from column ``shared_offset``; ``up`` [rows, heads * plain + heads * value] is the
    up-projection of the normalised latent.  The ``rot`` parts are rotated by the rows' positions
    (interleaved pairs); the cache gets per head the key ``[plain | rotated shared part]`` and the
    value.  ``value_dim`` (default: the cache's value size) is the size of a value in ``up``; a
    cache whose values are wider gets zeros behind them.  Returns the queries
    [rows, heads * (plain + rot)]."""
    _need(proj, "latent_assemble proj")
    _need(up, "latent_assemble up", proj.dtype)
    if kv.storage.dtype != proj.dtype or kv.n_kv != n_heads or kv.head_dim != plain + rot:
        raise KernelError(f"latent_assemble: the cache entry ({kv.n_kv} heads of {kv.head_dim}, {kv.storage.dtype}) does "
                          f"not fit {n_heads} heads of {plain} + {rot}, {proj.dtype}")
    value_dim = kv.v_dim if value_dim is None else int(value_dim)
    if value_dim > kv.v_dim:
        raise KernelError(f"latent_assemble: values of {value_dim} do not fit the cache's {kv.v_dim}")
    if proj.shape[0] != rows.n_rows or tuple(up.shape) != (rows.n_rows, n_heads * (plain + value_dim)):
        raise KernelError(f"latent_assemble: shapes proj {tuple(proj.shape)}, up {tuple(up.shape)} for {rows.n_rows} rows")
    if rot and (rotary is None or rotary.layout != "interleaved" or rotary.rotary_dim != rot):
        raise KernelError("latent_assemble: the rotated part needs interleaved tables of its size")
    q = torch.empty((rows.n_rows, n_heads * (plain + rot)), dtype=proj.dtype, device=proj.device)
    size = proj.element_size()
    _call("thn_latent_assemble", _ptr(q), proj.data_ptr() + q_offset * size, proj.shape[1],
          proj.data_ptr() + shared_offset * size, proj.shape[1], _ptr(up), _ptr(rotary.cos) if rot else None,
          _ptr(rotary.sin) if rot else None, rotary.cos.shape[0] if rot else 0, _ptr(rows.row_slot), _ptr(rows.row_pos),
          _ptr(kv.storage), _ptr(kv.block_table), kv.block_table.shape[1], kv.page_size, rows.n_rows, n_heads, plain, rot,
          kv.v_dim, value_dim, _code(proj, "latent_assemble"), _ptr(err), _stream())
    return q


# ------------------------------------------------------------------ matrix memory (mLSTM)


MLSTM_COLUMNS_PER_BLOCK = 16    # csrc/mlstm.cu: columns of a head's matrix per block (checked against the library)


def mlstm_column_blocks(value_dim: int) -> int:
    """Blocks of columns into which the recurrence kernel cuts a head's matrix; each keeps a
    copy of the head's normaliser state."""
    if lib().thn_mlstm_columns_per_block() != MLSTM_COLUMNS_PER_BLOCK:
        raise KernelError("mlstm: the kernel library was built with another number of columns per block")
    return -(-int(value_dim) // MLSTM_COLUMNS_PER_BLOCK)


def set_mlstm_kernel(staged: bool = True, lanes: int = 0) -> None:
    """Which kernel steps of several tokens take (tests and measurement): the one that stages
    tokens in shared memory or the plain one; 8, 16 or 32 lanes per column, or 0: by the step's size."""
    lib().thn_set_mlstm_staged(int(bool(staged)), int(lanes))


def mlstm(proj: torch.Tensor, gate_pre: torch.Tensor, bias_i: torch.Tensor, bias_f: torch.Tensor, cap: float,
          state: torch.Tensor, normaliser: torch.Tensor, rows: StepRows, n_heads: int, key_dim: int, value_dim: int,
          q_scale: float, floor: float = 1e-6) -> torch.Tensor:
    """The matrix-memory recurrence over a step's rows.  ``proj`` rows hold ``[q | k | v | ...]``
    (heads * key_dim, heads * key_dim, heads * value_dim); ``gate_pre`` float32 [rows, 2 * heads]
    the pre-activations of the input gates, then of the forget gates (biases are added here).
    ``state`` float32 [slots, heads, value_dim, key_dim] and ``normaliser`` float32
    [slots, heads, column blocks, key_dim + 1] (n, then m) are read and updated.  Returns the
    read-out float32 [rows, heads, value_dim].  Single-token steps run as one kernel."""
    _need(proj, "mlstm proj")
    _need(gate_pre, "mlstm gates", torch.float32)
    _need(bias_i, "mlstm bias", torch.float32)
    _need(bias_f, "mlstm bias", torch.float32)
    _need(state, "mlstm state", torch.float32)
    _need(normaliser, "mlstm normaliser", torch.float32)
    n = rows.n_rows
    blocks = mlstm_column_blocks(value_dim)
    if proj.shape[0] != n or tuple(gate_pre.shape) != (n, 2 * n_heads) or bias_i.shape[0] != n_heads \
            or bias_f.shape[0] != n_heads or tuple(state.shape[1:]) != (n_heads, value_dim, key_dim) \
            or tuple(normaliser.shape[1:]) != (n_heads, blocks, key_dim + 1) or normaliser.shape[0] != state.shape[0]:
        raise KernelError(f"mlstm: shapes proj {tuple(proj.shape)}, gates {tuple(gate_pre.shape)}, state "
                          f"{tuple(state.shape)}, normaliser {tuple(normaliser.shape)} do not fit {n_heads} heads of "
                          f"{key_dim} x {value_dim}")
    o = torch.empty((n, n_heads, value_dim), dtype=torch.float32, device=proj.device)
    raw = rows.max_q_len == 1
    gates = gate_pre
    if not raw:
        gates = torch.empty_like(gate_pre)
        _call("thn_mlstm_gates", _ptr(gates), _ptr(gate_pre), _ptr(bias_i), _ptr(bias_f), float(cap), n, n_heads, _stream())
    _call("thn_mlstm_recurrence", _ptr(o), _ptr(state), _ptr(normaliser), _ptr(proj), proj.shape[1], _ptr(gates),
          _ptr(bias_i), _ptr(bias_f), float(cap), int(raw), _ptr(rows.cu_seqlens), _ptr(rows.slots), rows.n_seqs, n_heads,
          key_dim, value_dim, float(q_scale), float(floor), _code(proj, "mlstm"), _stream())
    return o


# ------------------------------------------------------------------ mixture of experts


@dataclass
class Routing:
    dense: torch.Tensor           # float32 [rows, experts]: the weight of every expert, 0 where not chosen
    chosen: torch.Tensor          # int32 [rows, top]
    chosen_weight: torch.Tensor   # float32 [rows, top]


SCORINGS = {"softmax": 0, "logistic": 1}


def moe_route(logits: torch.Tensor, n_experts: int, n_groups: int, keep: int, top: int, scale: float,
              scoring: str = "softmax", renormalise: Optional[float] = None) -> Routing:
    """Routing weights from float32 router logits (the first ``n_experts`` columns of
    ``logits``): scores by softmax over all experts or (``scoring`` "logistic") the logistic
    function of each logit, the ``keep`` best of ``n_groups`` groups of neighbours (a group's
    score is its largest), the ``top`` best allowed experts, weights ``score * scale``.
    ``renormalise`` (a small number, softmax scores only): the chosen experts' scores are divided by
    their sum plus that number first."""
    _need(logits, "moe_route logits", torch.float32)
    rows = logits.shape[0]
    if logits.shape[1] < n_experts:
        raise KernelError(f"moe_route: rows of {logits.shape[1]} logits for {n_experts} experts")
    dense = torch.empty((rows, n_experts), dtype=torch.float32, device=logits.device)
    chosen = torch.empty((rows, top), dtype=torch.int32, device=logits.device)
    weight = torch.empty((rows, top), dtype=torch.float32, device=logits.device)
    _call("thn_moe_route", _ptr(dense), _ptr(chosen), _ptr(weight), _ptr(logits), logits.shape[1], rows, n_experts,
          n_groups, keep, top, float(scale), SCORINGS[scoring], int(renormalise is not None), float(renormalise or 0.0),
          _stream())
    return Routing(dense, chosen, weight)


def routed_clamped_glu(gu: torch.Tensor, routing: Routing, ff: int, shared_ff: int, limit: float, shared_limit: float,
                       alpha: float, shared_logit: Optional[torch.Tensor] = None, logit_column: int = 0,
                       weight_at: str = "input") -> torch.Tensor:
    """Experts ``g * logistic(alpha * g) * (u + 1)`` with ``g = min(w * gate, limit)`` and
    ``u = clamp(w * up, -limit, limit)``, ``w`` the routing weight of the column's expert: the
    expert sees the token times its weight, and its projections are linear.  ``gu`` [rows,
    2 * (experts * ff + shared_ff)] holds the gates of all columns, then the ups.  The shared
    expert's columns take ``w = 1`` and ``shared_limit`` and are multiplied by
    ``logistic(shared_logit[:, logit_column])`` (no gate without ``shared_logit``); columns of an
    expert that was not chosen are zero.  ``weight_at`` "output": the expert sees the token itself
    and ``w`` multiplies its activation instead.  Returns [rows, experts * ff + shared_ff]."""
    if weight_at not in ("input", "output"):
        raise KernelError(f"routed_clamped_glu: weight_at {weight_at!r} is neither 'input' nor 'output'")
    _need(gu, "routed_clamped_glu gu")
    rows, n_experts = routing.dense.shape
    width = n_experts * ff + shared_ff
    if tuple(gu.shape) != (rows, 2 * width):
        raise KernelError(f"routed_clamped_glu: gu is {tuple(gu.shape)}, expected {(rows, 2 * width)}")
    logit_ptr, stride = None, 0
    if shared_logit is not None:
        _need(shared_logit, "routed_clamped_glu gate logits", torch.float32)
        logit_ptr, stride = shared_logit.data_ptr() + 4 * logit_column, shared_logit.shape[1]
    out = torch.empty((rows, width), dtype=gu.dtype, device=gu.device)
    _call("thn_routed_clamped_glu", _ptr(out), _ptr(gu), _ptr(routing.dense), logit_ptr, stride, rows, n_experts, ff,
          shared_ff, float(limit), float(shared_limit or 1.0), float(alpha), int(weight_at == "output"),
          _code(gu, "routed_clamped_glu"), _stream())
    return out


def routed_gelu(u: torch.Tensor, routing: Routing, ff: int, shared_ff: int,
                shared_logit: Optional[torch.Tensor] = None, logit_column: int = 0) -> torch.Tensor:
    """u [rows, experts * ff + shared_ff] -> gelu(u) (the exact one) times the routing weight of
    the column's expert; the shared expert's columns times logistic(shared_logit[:, logit_column])
    (no gate without ``shared_logit``)."""
    _need(u, "routed_gelu u")
    rows, n_experts = routing.dense.shape
    if tuple(u.shape) != (rows, n_experts * ff + shared_ff):
        raise KernelError(f"routed_gelu: u is {tuple(u.shape)}, expected {(rows, n_experts * ff + shared_ff)}")
    logit_ptr, stride = None, 0
    if shared_logit is not None:
        _need(shared_logit, "routed_gelu gate logits", torch.float32)
        logit_ptr, stride = shared_logit.data_ptr() + 4 * logit_column, shared_logit.shape[1]
    out = torch.empty_like(u)
    _call("thn_routed_gelu", _ptr(out), _ptr(u), _ptr(routing.dense), logit_ptr, stride, rows, n_experts, ff, shared_ff,
          _code(u, "routed_gelu"), _stream())
    return out


# ------------------------------------------------------------------ hyper-connections


@dataclass
class StreamNumbers:
    """The numbers of one sublayer's hyper-connection (float32, on the device): ``read`` [streams]
    (how the sublayer's input is mixed from the streams), ``mix`` [streams, streams] ([from, to]) and
    ``write`` [streams] (how the streams are remixed and the sublayer's output added)."""

    read: torch.Tensor
    mix: torch.Tensor
    write: torch.Tensor


def hyper_norm(streams: Optional[torch.Tensor], n_streams: int, dtype: torch.dtype, *,
               start: Optional[torch.Tensor] = None, y: Optional[torch.Tensor] = None,
               written: Optional[StreamNumbers] = None, read: Optional[torch.Tensor] = None,
               gain: Optional[torch.Tensor] = None, eps: float = 1.0) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """Between two sublayers over a residual stream of ``n_streams`` copies kept in float32
    (``streams`` [rows, n_streams * width], updated in place): the write of the sublayer that
    produced ``y`` (``X'_i = sum_j mix[j, i] X_j + write[i] y``), then the read of the next one and
    its RMS norm, ``n = u / sqrt(mean(u^2) + eps) * gain`` with ``u = sum_j read[j] X'_j`` and
    ``gain`` float32 of one entry or ``[width]``.  ``start`` (float32 [rows, width]) instead of
    ``streams``: every stream starts as that row.  Returns ``(streams, n)``; ``n`` is None
    without ``read``."""
    if (streams is None) == (start is None):
        raise KernelError("hyper_norm: either the streams or the row they start as")
    if start is not None:
        _need(start, "hyper_norm start", torch.float32)
        streams = torch.empty((start.shape[0], n_streams * start.shape[1]), dtype=torch.float32, device=start.device)
    _need(streams, "hyper_norm streams", torch.float32)
    rows = streams.shape[0]
    if streams.dim() != 2 or streams.shape[1] % n_streams:
        raise KernelError(f"hyper_norm: streams {tuple(streams.shape)} are not {n_streams} rows side by side")
    width = streams.shape[1] // n_streams
    if y is not None:
        _need(y, "hyper_norm y", dtype)
        if written is None or tuple(y.shape) != (rows, width):
            raise KernelError(f"hyper_norm: y {tuple(y.shape)} for rows of {width}, with its numbers")
        _need(written.mix, "hyper_norm mix", torch.float32)
        _need(written.write, "hyper_norm write", torch.float32)
        if written.mix.numel() != n_streams * n_streams or written.write.numel() != n_streams:
            raise KernelError("hyper_norm: the numbers of the write do not fit the streams")
    n = None
    if read is not None:
        _need(read, "hyper_norm read", torch.float32)
        _need(gain, "hyper_norm gain", torch.float32)
        if read.numel() != n_streams or gain.numel() not in (1, width):
            raise KernelError("hyper_norm: the numbers of the read or the gain do not fit")
        n = torch.empty((rows, width), dtype=dtype, device=streams.device)
    _call("thn_hyper_norm", _ptr(n), _ptr(streams), _ptr(start), _ptr(y), _ptr(written.mix) if y is not None else None,
          _ptr(written.write) if y is not None else None, _ptr(read), _ptr(gain),
          int(gain is not None and gain.numel() != 1), float(eps), rows, width, n_streams, DTYPE_CODE[dtype], _stream())
    return streams, n


# ------------------------------------------------------------------ linear attention, selective scan


def linear_attention(proj: torch.Tensor, offsets: Tuple[int, int, int], state: torch.Tensor, rows: StepRows,
                     n_heads: int, key_dim: int, value_dim: int, *, decay: Optional[torch.Tensor] = None,
                     gate: Optional[torch.Tensor] = None, gate_bias: Optional[torch.Tensor] = None, tau: float = 1.0,
                     q_scale: float = 1.0, silu_inputs: bool = False) -> torch.Tensor:
    """Linear attention with a decayed matrix state over a step's rows: per head
    ``S <- diag(a) S + k v^T``, ``o = S^T q * q_scale`` from the state the sequences' earlier steps
    left.  ``proj`` rows hold q, k (``heads * key_dim``) and v (``heads * value_dim``) from the
    columns ``offsets``; with ``silu_inputs`` they pass silu first.  The decay is ``decay`` (float32
    ``[heads]``, one constant per head) or, per token and key channel,
    ``logistic(gate + gate_bias) ** (1 / tau)`` with ``gate`` float32 ``[rows, >= heads * key_dim]``.
    ``state`` float32 [slots, heads, value_dim, key_dim] is read and updated.  Returns the read-out,
    float32 [rows, heads, value_dim].  Two kernels: the inputs' activations and the decays once per
    entry into float32 scratch rows, then the recurrence."""
    _need(proj, "linear_attention proj")
    _need(state, "linear_attention state", torch.float32)
    if (decay is None) == (gate is None):
        raise KernelError("linear_attention: either a constant decay per head or a gate per token")
    if proj.shape[0] != rows.n_rows or tuple(state.shape[1:]) != (n_heads, value_dim, key_dim):
        raise KernelError(f"linear_attention: proj {tuple(proj.shape)}, state {tuple(state.shape)} do not fit {n_heads} "
                          f"heads of {key_dim} x {value_dim} over {rows.n_rows} rows")
    if decay is not None:
        _need(decay, "linear_attention decay", torch.float32)
        if decay.shape[0] != n_heads:
            raise KernelError(f"linear_attention: {decay.shape[0]} decays for {n_heads} heads")
    else:
        _need(gate, "linear_attention gate", torch.float32)
        if gate.shape[0] != rows.n_rows or gate.shape[1] < n_heads * key_dim:
            raise KernelError(f"linear_attention: gate {tuple(gate.shape)}")
        if gate_bias is not None:
            _need(gate_bias, "linear_attention gate bias", torch.float32)
            if gate_bias.shape[0] != n_heads * key_dim:
                raise KernelError(f"linear_attention: gate bias {tuple(gate_bias.shape)}")
    o = torch.empty((rows.n_rows, n_heads, value_dim), dtype=torch.float32, device=proj.device)
    mode = 0 if decay is not None else 1
    scratch = torch.empty(lib().thn_linear_attention_scratch_floats(rows.n_rows, n_heads, key_dim, value_dim, mode),
                          dtype=torch.float32, device=proj.device)
    _call("thn_linear_attention", _ptr(o), _ptr(state), _ptr(scratch), _ptr(proj), proj.shape[1], int(offsets[0]), int(offsets[1]),
          int(offsets[2]), _ptr(decay), _ptr(gate), gate.shape[1] if gate is not None else 0, _ptr(gate_bias), float(tau),
          _ptr(rows.cu_seqlens), _ptr(rows.slots), rows.n_rows, rows.n_seqs, n_heads, key_dim, value_dim, float(q_scale),
          0 if decay is not None else 1, int(bool(silu_inputs)), _code(proj, "linear_attention"), _stream())
    return o


def causal_conv(proj: torch.Tensor, offset: int, channels: int, weight: torch.Tensor, bias: Optional[torch.Tensor],
                ring: torch.Tensor, rows: StepRows, seq_lens: torch.Tensor) -> torch.Tensor:
    """A short causal convolution per channel over time, then silu: ``out[t, c] = silu(bias[c] +
    sum_j weight[c, j] raw[t - (taps - 1) + j, c])`` with zeros before a sequence's start; the raw
    inputs are the columns ``[offset, offset + channels)`` of ``proj``.  Inputs of earlier steps
    come from ``ring`` [slots, taps, channels] (position p at ``p mod taps``), which
    :func:`conv_ring_update` brings up to date after this call; ``seq_lens`` holds the tokens each
    slot held before the step."""
    _need(proj, "causal_conv proj")
    _need(weight, "causal_conv weight", torch.float32)
    _need(ring, "causal_conv ring", proj.dtype)
    taps = weight.shape[1]
    if tuple(weight.shape) != (channels, taps) or tuple(ring.shape[1:]) != (taps, channels) or proj.shape[0] != rows.n_rows \
            or offset + channels > proj.shape[1]:
        raise KernelError(f"causal_conv: proj {tuple(proj.shape)}, weight {tuple(weight.shape)}, ring {tuple(ring.shape)}")
    if bias is not None:
        _need(bias, "causal_conv bias", torch.float32)
    out = torch.empty((rows.n_rows, channels), dtype=proj.dtype, device=proj.device)
    _call("thn_causal_conv", _ptr(out), _ptr(proj), proj.shape[1], int(offset), _ptr(weight), _ptr(bias), _ptr(ring),
          _ptr(rows.row_slot), _ptr(rows.row_pos), _ptr(seq_lens), rows.n_rows, channels, taps, _code(proj, "causal_conv"),
          _stream())
    return out


def conv_ring_update(ring: torch.Tensor, proj: torch.Tensor, offset: int, rows: StepRows, seq_lens: torch.Tensor) -> None:
    """The step's last raw inputs (at most ``taps`` per sequence) go into ``ring``."""
    _need(ring, "conv_ring_update ring", proj.dtype)
    _call("thn_conv_ring_update", _ptr(ring), _ptr(proj), proj.shape[1], int(offset), _ptr(rows.cu_seqlens), _ptr(rows.slots),
          _ptr(seq_lens), rows.n_seqs, ring.shape[2], ring.shape[1], _code(proj, "conv_ring_update"), _stream())


def selective_scan(x: torch.Tensor, dt_pre: torch.Tensor, dt_bias: torch.Tensor, bc: torch.Tensor, a: torch.Tensor,
                   d: torch.Tensor, gate: torch.Tensor, gate_offset: int, state: torch.Tensor, rows: StepRows) -> torch.Tensor:
    """The selective scan over a step's rows: per channel c and state entry n
    ``S[c, n] <- exp(dt_c a[c, n]) S[c, n] + dt_c x_c B_n``, ``y_c = (sum_n S[c, n] C_n + d_c x_c) *
    silu(z_c)`` with ``dt = softplus(dt_pre + dt_bias)`` (float32), ``bc`` rows ``[B | C]`` and z the
    columns of ``gate`` from ``gate_offset``.  ``state`` float32 [slots, channels, n] is read and
    updated.  Returns y [rows, channels] of the activation type."""
    _need(x, "selective_scan x")
    _need(dt_pre, "selective_scan dt", torch.float32)
    _need(dt_bias, "selective_scan dt bias", torch.float32)
    _need(bc, "selective_scan bc", x.dtype)
    _need(a, "selective_scan a", torch.float32)
    _need(d, "selective_scan d", torch.float32)
    _need(gate, "selective_scan gate", x.dtype)
    _need(state, "selective_scan state", torch.float32)
    n_rows, channels = x.shape
    n_state = a.shape[1]
    if n_rows != rows.n_rows or tuple(dt_pre.shape) != (n_rows, channels) or tuple(a.shape) != (channels, n_state) \
            or bc.shape[0] != n_rows or bc.shape[1] < 2 * n_state or tuple(state.shape[1:]) != (channels, n_state) \
            or gate.shape[0] != n_rows or gate_offset + channels > gate.shape[1] or d.shape[0] != channels \
            or dt_bias.shape[0] != channels:
        raise KernelError(f"selective_scan: x {tuple(x.shape)}, dt {tuple(dt_pre.shape)}, bc {tuple(bc.shape)}, a "
                          f"{tuple(a.shape)}, state {tuple(state.shape)}, gate {tuple(gate.shape)} from {gate_offset}")
    y = torch.empty_like(x)
    _call("thn_selective_scan", _ptr(y), _ptr(state), _ptr(x), _ptr(dt_pre), _ptr(dt_bias), _ptr(bc), bc.shape[1], _ptr(a),
          _ptr(d), gate.data_ptr() + gate_offset * gate.element_size(), gate.shape[1], _ptr(rows.cu_seqlens),
          _ptr(rows.slots), rows.n_seqs, channels, n_state, _code(x, "selective_scan"), _stream())
    return y


def rotate_gate(a: torch.Tensor, gate: torch.Tensor, gate_offset: int, n_heads: int, size: int,
                rotary: Optional[RotaryTables], rows: StepRows, err: Optional[torch.Tensor], scale: float = 1.0,
                out: Optional[torch.Tensor] = None, out_offset: int = 0) -> torch.Tensor:
    """``a`` [rows, heads * size], every head turned back by its row's position (the inverse of the
    turn that :func:`qk_prepare` gave the values; ``rotary`` None: no turn), times
    ``logistic(gate[:, gate_offset : gate_offset + heads * size])`` times ``scale``.  With ``out`` the
    result goes to its columns from ``out_offset``."""
    _need(a, "rotate_gate a")
    _need(gate, "rotate_gate gate", a.dtype)
    n_rows, width = a.shape
    if width != n_heads * size or gate.shape[0] != n_rows or gate_offset + width > gate.shape[1]:
        raise KernelError(f"rotate_gate: a {tuple(a.shape)}, gate {tuple(gate.shape)} from {gate_offset}")
    if out is None:
        out, out_offset = torch.empty_like(a), 0
    else:
        _need(out, "rotate_gate out", a.dtype)
        if out.shape[0] != n_rows or out_offset < 0 or out_offset + width > out.shape[1]:
            raise KernelError(f"rotate_gate: out {tuple(out.shape)} has no room for {width} columns from {out_offset}")
    _call("thn_rotate_gate", out.data_ptr() + out_offset * out.element_size(), out.shape[1], _ptr(a),
          gate.data_ptr() + gate_offset * gate.element_size(), gate.shape[1], _ptr(rotary.cos) if rotary else None,
          _ptr(rotary.sin) if rotary else None, rotary.cos.shape[0] if rotary else 0, rotary.rotary_dim if rotary else 0,
          ROTARY_LAYOUTS[rotary.layout] if rotary else 0, _ptr(rows.row_pos), n_rows, n_heads, size, float(scale),
          _code(a, "rotate_gate"), _ptr(err), _stream())
    return out


# ------------------------------------------------------------------ token choice


def choose_tokens(logits: torch.Tensor, temperature: Optional[torch.Tensor] = None,
                  seed: Optional[torch.Tensor] = None, stream_id: Optional[torch.Tensor] = None,
                  step: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                  slots: Optional[torch.Tensor] = None, last_token: Optional[torch.Tensor] = None,
                  bump_step: bool = False) -> torch.Tensor:
    """logits float32 [rows, vocab] -> int32 [rows].  Rows with temperature 0 (or no
    temperature tensor at all) take the argmax, lowest index on ties; others are drawn
    from softmax(logits / T) with Philox noise keyed by (seed, stream, step) of the row.
    With ``slots`` the per-row values are per-sequence state indexed by ``slots[row]``;
    ``last_token`` (same indexing) also receives the choice; ``bump_step`` increments the
    step counter after use."""
    _need(logits, "choose_tokens logits", torch.float32)
    rows, vocab = logits.shape
    if out is None:
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    if temperature is not None:
        _need(temperature, "temperature", torch.float32)
        _need(seed, "seed", torch.int64)
        _need(stream_id, "stream", torch.int32)
        _need(step, "step", torch.int32)
    need = lib().thn_choose_tokens_scratch_floats(rows, vocab)
    scratch = torch.empty(need, dtype=torch.float32, device=logits.device) if need else None
    _call("thn_choose_tokens", _ptr(out), _ptr(logits), rows, vocab, logits.stride(0), _ptr(temperature),
          _ptr(seed), _ptr(stream_id), _ptr(step), _ptr(slots), _ptr(last_token), int(bump_step), _ptr(scratch),
          _stream())
    return out


def gather_i32(src: torch.Tensor, index: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _need(src, "gather_i32 src", torch.int32)
    _need(index, "gather_i32 index", torch.int32)
    if out is None:
        out = torch.empty(index.shape[0], dtype=torch.int32, device=src.device)
    _call("thn_gather_i32", _ptr(out), _ptr(src), _ptr(index), index.shape[0], _stream())
    return out


__all__ = [
    "KernelError", "KernelLibraryError", "KVView", "RotaryTables", "RowTiles", "StepRows", "row_tiles_of", "prompt_attention_tile", "linear_stream", "linear_swiglu", "linear_tcgen05", "add_rmsnorm", "advance",
    "ROW_TILE", "attention", "attention_decode_bf16", "attention_generic", "attention_prefill_bf16", "attention_prefill_tcgen05", "decode_splits", "choose_tokens", "gather_i32", "gather_rows", "lib", "linear", "new_error_word",
    "qk_norm_rope_cache", "qk_prepare", "Gain", "STREAM_AS_IS", "residual_norm", "gather_rows_scaled", "logistic_gate", "latent_norm", "latent_assemble", "mlstm", "mlstm_column_blocks", "set_mlstm_kernel", "Routing", "moe_route", "routed_gelu", "gated_head_norm", "clamped_glu", "routed_clamped_glu", "polynorm", "scale_", "ScoreShape", "PLAIN_SCORES", "DeltaShape", "delta_rule", "qkv_attention", "raise_on_device_error", "rmsnorm", "StreamNumbers", "hyper_norm", "linear_attention", "causal_conv", "conv_ring_update", "selective_scan", "rotate_gate", "rope_table", "scatter_i32", "step_rows", "swiglu",
]
