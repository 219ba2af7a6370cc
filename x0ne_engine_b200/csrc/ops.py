"""Python entry points of the CUDA kernels: argument checks, then one C call each.

Tensors are torch CUDA tensors; a kernel gets raw device pointers and runs on torch's current
stream, so calls order themselves with torch work and can be captured into a CUDA graph.
Every function raises `KernelError` when the C entry point refuses its arguments or the launch
fails; nothing here computes on the CPU or through another library.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import Structure, c_float, c_int, c_int32, c_int64, c_void_p
from typing import Optional

import torch

from . import build as _build

F32, BF16 = 0, 1


class KernelError(RuntimeError):
    pass


def dtype_tag(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"no kernel for dtype {dtype}")


class PagedCacheArg(Structure):
    """Mirror of `struct PagedCache` in common.cuh."""
    _fields_ = [("base", c_void_p), ("page_table", c_void_p), ("page_stride", c_int64),
                ("table_stride", c_int32), ("ring_pages", c_int32), ("page_size", c_int32),
                ("kv_heads", c_int32), ("head_dim", c_int32), ("n_pages", c_int32), ("v_dim", c_int32)]

    @property
    def value_dim(self) -> int:
        """Width of a cached value row (0 when the page keeps no values)."""
        return self.head_dim if self.v_dim == 0 else max(int(self.v_dim), 0)


class AttnExtraArg(Structure):
    """Mirror of `struct AttnExtra` in common.cuh: what an attention kernel is asked for beyond causal
    softmax over a window (all zero: nothing)."""
    _fields_ = [("chunk", c_int32), ("v_from_k", c_int32), ("sink", c_void_p), ("gate", c_void_p),
                ("gate_ld", c_int64), ("q_ld", c_int64), ("keep_first", c_int32), ("gate_wide", c_int32), ("slope", c_void_p), ("out_f32", c_int32)]


def attn_extra(chunk: int = 0, v_from_k: int = 0, sink: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None,
               gate_ld: int = 0, q_ld: int = 0, keep_first: int = 0, gate_wide: bool = False,
               slope: Optional[torch.Tensor] = None, out_f32: bool = False) -> AttnExtraArg:
    """`sink`: float32 per q head.  `gate`: a view whose element (row, head) lies at row * gate_ld + head; with
    `gate_wide` it holds a value per (row, head, value) at row * gate_ld + head * value width + value.
    `keep_first`: the keys at positions below it stay visible to every later query, whatever the window or chunk.
    `slope`: float32 per q head; slope[h] * (i - j) is taken off the scaled score of query i and key j.
    `out_f32`: the results are written as float32 (the output tensor is float32) whatever the queries' type."""
    if sink is not None:
        _need(sink, torch.float32, "sink")
    if slope is not None:
        _need(slope, torch.float32, "distance slopes")
    return AttnExtraArg(int(chunk or 0), int(v_from_k or 0), _ptr(sink), _ptr(gate), int(gate_ld), int(q_ld), int(keep_first or 0),
                        1 if gate_wide else 0, _ptr(slope), 1 if out_f32 else 0)


class SsmArg(Structure):
    """Mirror of `struct SsmArgs` in ssm.cu."""
    _fields_ = [("u", c_void_p), ("xz", c_void_p), ("xz_ld", c_int64), ("z_col", c_int32), ("dt_raw", c_void_p), ("dt_bias", c_void_p),
                ("A", c_void_p), ("bc", c_void_p), ("bc_ld", c_int64), ("b_col", c_int32), ("c_col", c_int32), ("D", c_void_p),
                ("out", c_void_p), ("state", c_void_p), ("state_stride", c_int64), ("conv_off", c_int64), ("seq_first_row", c_void_p),
                ("seq_slot", c_void_p), ("channels", c_int32), ("N", c_int32), ("taps", c_int32)]


class SampleIOArg(Structure):
    """Mirror of `struct SampleIO` in sampling.cu."""
    _fields_ = [("logits", c_void_p), ("temperature", c_void_p), ("top_p", c_void_p), ("seed", c_void_p),
                ("draw_counter", c_void_p), ("stop_ids", c_void_p), ("finished", c_void_p), ("budget", c_void_p),
                ("out_token", c_void_p), ("next_token", c_void_p), ("next_pos", c_void_p),
                ("status", c_void_p), ("row_best", c_void_p), ("ld", c_int64), ("vocab", c_int32), ("n_stop", c_int32)]


_libs = {}


_P, _I, _F, _L = c_void_p, c_int, c_float, c_int64
# Argument types of the entry points, declared once per library: ctypes then converts plain Python
# numbers itself, which is about a third of the cost of building a c_int or c_void_p per argument
# and per call (1.4 us against 3.8 us for ten arguments).  Pointers are passed as integers.
_SIGNATURES = {
    "x0ne_embedding": [_P, _I, _P, _P, _I, _I, _I, _F, _P],
    "x0ne_add_normed_rmsnorm": [_P, _P, _P, _F, _P, _P, _I, _P, _I, _I, _F, _P],
    "x0ne_whole_norm_rope_kv_write": [_P, _I, _I, _I, _I, _P, _P, _F, _P, _I, _P, _I, _P, _I, None, _P, _P, _I, _I, _P],
    "x0ne_relu2": [_P, _P, _I, _L, _P],
    "x0ne_moe_route": [_P, _I, _P, _I, _I, _I, _I, _I, _P, _P, _P, _I, _I, _I, _I, _F, _P],
    "x0ne_rope_pairs_kv_write": [_P, _I, _I, _I, _I, _P, _P, _I, _I, _I, _I, _F, _P, _I, _I, None, _P, _P, _I, _I, _P],
    "x0ne_diff_heads": [_P, _P, _L, _P, _I, _I, _I, _I, _F, _F, _F, _P],
    "x0ne_causal_conv_silu": [_P, _L, _I, _P, _P, _P, _L, _L, _P, _P, _P, _I, _I, _I, _P],
    "x0ne_selective_scan": ["ssm", _I, _I, _I, _P],
    "x0ne_add2_group_rmsnorm": [_P, _P, _P, _P, _P, _I, _P, _I, _I, _I, _F, _P],
    "x0ne_open_pass": [_P, _P, _I, _P, _I, _P, _F, _P, _I, _I, _I, _P],
    "x0ne_head_norm_kv_write": [_P, _I, _I, _I, _I, _P, _P, _F, _F, _I, _I, _P, _I, None, _P, _P, _I, _P],
    "x0ne_bias_act": [_P, _P, _P, _I, _I, _I, _I, _F, _F, _P],
    "x0ne_token_shift_mix": [_P, _I, _P, _I, _P, _L, _P, _L, _L, _P, _P, _I, _I, _P],
    "x0ne_wkv_scan": [_P, _P, _P, _I, _P, _P, _P, _P, _P, _P, _L, _P, _P, _I, _I, _I, _I, _I, _P],
    "x0ne_head_norm_gate": [_P, _P, _P, _P, _I, _I, _I, _I, _F, _P],
    "x0ne_tanh_rows": [_P, _P, _I, _L, _P],
    "x0ne_moe_group": [_P, _I, _I, _P, _P, _P, _I, _I, _P, _P],
    "x0ne_moe_gather_rows": [_P, _I, _P, _P, _I, _I, _P, _I, _P],
    "x0ne_moe_product_tc": [_I, _P, _L, _P, _I, _I, _I, _P, _P, _P, _I, _P, _P, _P],
    "x0ne_moe_product": [_I, _P, _L, _P, _I, _I, _I, _P, _P, _I, _I, _P, _I, _P],
    "x0ne_moe_combine": [_P, _P, _I, _P, _P, _I, _I, _P, _P, _P, _I, _I, _P],
    "x0ne_add_rmsnorm": [_P, _P, _P, _P, _I, _P, _I, _I, _F, _P],
    "x0ne_add2_rmsnorm": [_P, _P, _P, _P, _P, _I, _P, _I, _I, _F, _P],
    "x0ne_glu_clipped": [_P, _P, _I, _I, _I, _F, _F, _F, _P],
    "x0ne_kv_write_blend": [_P, _I, _I, _I, _I, _P, _P, _I, None, _P, _P, _I, _P],
    "x0ne_latent_prepare": [_P, _I, _I, _I, _P, _L, _P, _F, _P, _F, _P, _I, _P, _I, _I, _I, _I, None, _P, _P, _I, _I, _P],
    "x0ne_attention_rows_ex": [_P, _P, _I, None, _P, _P, _I, _I, _F, _I, "ex", _P],
    "x0ne_gemm_f32_nt_batched": [_P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _L, _L, _L, _P],
    "x0ne_attention_flex_prefill": [_P, _P, None, _P, _P, _I, _P, _P, _P, _I, _F, _I, "ex", _P],
    "x0ne_attention_flex_decode": [_P, _P, None, _P, _P, _I, _I, _F, _I, "ex", _I, _P, _L, _P],
    "x0ne_qk_norm_rope_kv_write": [_P, _I, _P, _P, _P, _I, _P, None, _P, _P, _I, _I, _F, _I, _P, _I, _P],
    "x0ne_swiglu": [_P, _P, _I, _I, _I, _P],
    "x0ne_attention_rows": [_P, _P, _I, None, _P, _P, _I, _I, _F, _I, _P],
    "x0ne_gemm_f32_nt": [_P, _P, _P, _I, _I, _I, _I, _I, _I, _P],
    "x0ne_attention_prefill_bf16": [_P, _P, None, _P, _P, _I, _P, _P, _P, _I, _F, _I, _P],
    "x0ne_attention_decode_bf16": [_P, _P, None, _P, _P, _I, _I, _F, _I, _I, _P, _L, _P],
    "x0ne_attention_decode_grouped_bf16": [_P, _P, None, _P, _P, _I, _I, _F, _I, _I, _I, _P, _L, _P],
    "x0ne_gemm_bf16_smallm": [_P, _P, _P, _I, _I, _I, _I, _I, _I, _P],
    "x0ne_gemm_bf16_smallm_glu": [_P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _F, _F, _P],
    "x0ne_gemm_bf16_tcgen05_glu": [_P, _P, _P, _I, _I, _I, _I, _I, _I, _P, _F, _F, _F, _P],
    "x0ne_gemm_bf16_skinny_tcgen05_glu": [_P, _P, _I, _P, _I, _I, _I, _I, _I, _P, _F, _F, _F, _P],
    "x0ne_attention_prefill_tcgen05": [_P, _P, _I, None, _P, _P, _I, _P, _P, _P, _I, _F, _I, _P, _P],
    "x0ne_gemm_bf16_tcgen05": [_P, _P, _P, _I, _I, _I, _I, _I, _I, _P, _P],
    "x0ne_gemm_bf16_skinny_tcgen05": [_P, _P, _I, _P, _I, _I, _I, _I, _I, _P, _P],
    "x0ne_sample": ["io", _I, _P],
    "x0ne_plan_pass": [_I, _P, _P, _P, _P, _L, _L, _P, _I, _I, _I, _P, _L, _P],
}


def _lib(name: str) -> ctypes.CDLL:
    lib = _libs.get(name)
    if lib is None:
        lib = _build.load(name)
        lib.x0ne_last_error.restype = ctypes.c_char_p
        for fn_name, args in _SIGNATURES.items():
            fn = getattr(lib, fn_name, None)
            if fn is not None:
                # None: the cache view, by value; "io": the sampler's arguments, by value
                fn.argtypes = [PagedCacheArg if a is None else SampleIOArg if a == "io" else AttnExtraArg if a == "ex" else SsmArg if a == "ssm" else a
                               for a in args]
                fn.restype = c_int
        _libs[name] = lib
    return lib


def loaded_libraries():
    """Paths of the kernel libraries this process has loaded."""
    return [lib._name for lib in _libs.values()]


LAUNCHES = 0   # kernel entry points called by this process (one or a few launches each)


def _check(lib, code: int, what: str) -> None:
    global LAUNCHES
    LAUNCHES += 1
    if code != 0:
        msg = lib.x0ne_last_error()
        raise KernelError(f"{what}: {msg.decode() if msg else 'error'} (code {code})")


def _stream() -> int:
    """The current stream of the current device, as a raw handle (the private accessor is some
    forty times cheaper than building a torch.cuda.Stream object for every launch)."""
    raw = getattr(torch._C, "_cuda_getCurrentRawStream", None)
    if raw is not None:
        return raw(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _need(t: torch.Tensor, dtype, what: str) -> None:
    if not t.is_cuda:
        raise KernelError(f"{what} is not on the GPU")
    if t.dtype != dtype:
        raise KernelError(f"{what} is {t.dtype}, the kernel needs {dtype}")
    if not t.is_contiguous():
        raise KernelError(f"{what} is not contiguous")


def plan_pass(slots, starts, first_row, tokens, r0: int, r1: int, want_sorted, tile_rows: int, launch_rows: int,
              stage: torch.Tensor):
    """Fills the pinned staging table `stage` (int32 [9][stride]) for rows [r0, r1) of a step (native
    host code, step_plan.cu).  `slots`, `starts` (int32 per sequence), `first_row` (int64, one more
    than sequences), `tokens` (int32, all rows of the step) and `want_sorted` (int64) are contiguous
    NumPy arrays.  Returns (sequences in the pass, tiles, most rows of one sequence, one more than the
    largest position, lo, hi) with want_sorted[lo:hi] the wanted rows of the pass."""
    lib = _lib("core")
    out = (c_int32 * 6)()
    code = lib.x0ne_plan_pass(len(slots), slots.ctypes.data, starts.ctypes.data, first_row.ctypes.data,
                              tokens.ctypes.data, r0, r1, want_sorted.ctypes.data, len(want_sorted), tile_rows,
                              launch_rows, stage.data_ptr(), stage.stride(0), ctypes.addressof(out))
    if code != 0:
        msg = lib.x0ne_last_error()
        raise KernelError(f"plan_pass: {msg.decode() if msg else 'error'} (code {code})")
    return tuple(out)


def embedding(table: torch.Tensor, tokens: torch.Tensor, resid: torch.Tensor, n_rows: int, scale: float = 1.0) -> None:
    """resid[r] = float32(table[tokens[r]]) * scale; an id outside the table gives a zero row."""
    lib = _lib("core")
    _need(tokens, torch.int32, "tokens")
    _need(resid, torch.float32, "residual")
    _need(table, table.dtype, "embedding table")
    vocab, hidden = table.shape
    if resid.shape[-1] != hidden or resid.numel() < n_rows * hidden or tokens.numel() < n_rows:
        raise KernelError("embedding: buffers are smaller than the rows asked for")
    _check(lib, lib.x0ne_embedding(_ptr(table), dtype_tag(table.dtype), _ptr(tokens), _ptr(resid),
                                   n_rows, hidden, vocab, float(scale), _stream()), "embedding")


def add_rmsnorm(resid: torch.Tensor, delta, weight: torch.Tensor, out: torch.Tensor,
                n_rows: int, eps: float, rows: Optional[torch.Tensor] = None, groups: int = 1) -> None:
    """resid += delta (if given); out = rmsnorm(resid) * weight.  `rows` gathers source rows.  `delta` may
    be a pair of tensors, the results of two branches that read the same normed rows: their float32
    sum is added.  `groups` > 1: a row is that many equal consecutive parts, each normed by its own root mean square."""
    lib = _lib("core")
    delta2 = None
    if isinstance(delta, (tuple, list)):
        parts = [d for d in delta if d is not None]
        if len(parts) > 2:
            raise KernelError("add_rmsnorm: at most two deltas")
        delta = parts[0] if parts else None
        delta2 = parts[1] if len(parts) > 1 else None
    hidden = weight.numel()
    _need(resid, torch.float32, "residual")
    _need(weight, torch.float32, "norm weight")
    _need(out, out.dtype, "norm output")
    if delta is not None:
        _need(delta, out.dtype, "delta")
        if delta.shape[-1] != hidden:
            raise KernelError("add_rmsnorm: delta width differs from the norm's")
    if rows is not None:
        _need(rows, torch.int32, "row list")
        if rows.numel() < n_rows:
            raise KernelError("add_rmsnorm: row list shorter than the rows asked for")
    elif resid.numel() < n_rows * hidden:
        raise KernelError("add_rmsnorm: residual smaller than the rows asked for")
    if resid.shape[-1] != hidden or out.shape[-1] != hidden or out.numel() < n_rows * hidden:
        raise KernelError("add_rmsnorm: widths differ or output too small")
    if delta2 is not None:
        _need(delta2, out.dtype, "second delta")
        if delta2.shape[-1] != hidden:
            raise KernelError("add_rmsnorm: delta width differs from the norm's")
    if groups != 1:
        if groups < 1 or hidden % groups:
            raise KernelError(f"add_rmsnorm: rows of {hidden} values do not split into {groups} equal parts")
        _check(lib, lib.x0ne_add2_group_rmsnorm(_ptr(resid), _ptr(delta), _ptr(delta2), _ptr(weight), _ptr(out), dtype_tag(out.dtype),
                                                _ptr(rows), n_rows, hidden, groups, eps, _stream()), "add_rmsnorm")
        return
    if delta2 is not None:
        _check(lib, lib.x0ne_add2_rmsnorm(_ptr(resid), _ptr(delta), _ptr(delta2), _ptr(weight), _ptr(out), dtype_tag(out.dtype),
                                          _ptr(rows), n_rows, hidden, eps, _stream()), "add_rmsnorm")
        return
    _check(lib, lib.x0ne_add_rmsnorm(_ptr(resid), _ptr(delta), _ptr(weight), _ptr(out), dtype_tag(out.dtype),
                                     _ptr(rows), n_rows, hidden, eps, _stream()), "add_rmsnorm")


def add_normed_rmsnorm(resid: torch.Tensor, delta: torch.Tensor, delta_weight: torch.Tensor, delta_eps: float,
                       weight: torch.Tensor, out: torch.Tensor, n_rows: int, eps: float,
                       rows: Optional[torch.Tensor] = None) -> None:
    """resid += rmsnorm(delta) * delta_weight (float32, never rounded); out = rmsnorm(resid) * weight.  `rows`
    gathers source rows."""
    lib = _lib("core")
    hidden = weight.numel()
    _need(resid, torch.float32, "residual")
    _need(weight, torch.float32, "norm weight")
    _need(delta_weight, torch.float32, "norm weight of the delta")
    _need(out, out.dtype, "norm output")
    _need(delta, out.dtype, "delta")
    if delta.shape[-1] != hidden or delta_weight.numel() != hidden or resid.shape[-1] != hidden or out.shape[-1] != hidden \
            or out.numel() < n_rows * hidden:
        raise KernelError("add_normed_rmsnorm: widths differ or output too small")
    if rows is not None:
        _need(rows, torch.int32, "row list")
        if rows.numel() < n_rows:
            raise KernelError("add_normed_rmsnorm: row list shorter than the rows asked for")
    elif resid.numel() < n_rows * hidden or delta.numel() < n_rows * hidden:
        raise KernelError("add_normed_rmsnorm: residual or delta smaller than the rows asked for")
    _check(lib, lib.x0ne_add_normed_rmsnorm(_ptr(resid), _ptr(delta), _ptr(delta_weight), delta_eps, _ptr(weight), _ptr(out),
                                            dtype_tag(out.dtype), _ptr(rows), n_rows, hidden, eps, _stream()),
           "add_normed_rmsnorm")


def whole_norm_rope_kv_write(src: torch.Tensor, k_col: int, v_col: int, q_norm: torch.Tensor, k_norm: Optional[torch.Tensor],
                             eps: float, freq: Optional[torch.Tensor], rot: int, table: Optional[torch.Tensor],
                             q_out: torch.Tensor, q_heads: int, cache: PagedCacheArg, row_slot: torch.Tensor,
                             row_pos: torch.Tensor, n_rows: int, write_kv: bool = True) -> None:
    """Queries and keys normed over their whole projection (one weight per projected value), rotated (the
    first `rot` values of every head, value i with i + rot/2), queries to `q_out`, keys and values into the
    cache.  `src` rows hold the queries at column 0, the keys at k_col, the values at v_col; with
    write_kv False only the queries are made (a layer that reads another layer's keys and values)."""
    lib = _lib("core")
    _need(src, src.dtype, "projection rows")
    _need(q_out, src.dtype, "q output")
    _need(row_slot, torch.int32, "row slots")
    _need(row_pos, torch.int32, "row positions")
    _need(q_norm, torch.float32, "q norm weight")
    qn = q_heads * cache.head_dim
    if q_norm.numel() != qn or q_out.shape[-1] != qn or q_out.numel() < n_rows * qn or src.numel() < n_rows * src.shape[-1]:
        raise KernelError("whole_norm_rope: widths or rows do not match")
    if write_kv:
        _need(k_norm, torch.float32, "k norm weight")
        if k_norm.numel() != cache.kv_heads * cache.head_dim:
            raise KernelError("whole_norm_rope: the key norm weight does not match the key projection")
    positions = 0
    if rot:
        _need(freq, torch.float32, "rotary frequencies")
        if freq.numel() * 2 != rot:
            raise KernelError("whole_norm_rope: frequencies are not rot / 2")
        if table is not None:
            _need(table, torch.float32, "rotary table")
            if table.dim() != 2 or table.shape[1] != rot:
                raise KernelError("whole_norm_rope: the table is not [positions, rot]")
            positions = table.shape[0]
    _check(lib, lib.x0ne_whole_norm_rope_kv_write(
        _ptr(src), dtype_tag(src.dtype), src.shape[-1], k_col, v_col, _ptr(q_norm), _ptr(k_norm) if write_kv else None, eps,
        _ptr(freq) if rot else None, rot, _ptr(table) if rot else None, positions, _ptr(q_out), q_heads, cache, _ptr(row_slot),
        _ptr(row_pos), n_rows, 1 if write_kv else 0, _stream()), "whole_norm_rope_kv_write")


def relu2(x: torch.Tensor, out: torch.Tensor, n_rows: int) -> None:
    """out = max(x, 0)^2 on the first n_rows rows."""
    lib = _lib("core")
    _need(x, x.dtype, "activation input")
    _need(out, x.dtype, "activation output")
    width = x.shape[-1]
    if out.shape[-1] != width or x.numel() < n_rows * width or out.numel() < n_rows * width:
        raise KernelError("relu2: widths or rows do not match")
    _check(lib, lib.x0ne_relu2(_ptr(x), _ptr(out), dtype_tag(x.dtype), n_rows * width, _stream()), "relu2")


# ---------------------------------------------------------------------------------------------
# routed feed-forward (csrc/moe.cu, module `core`; the tensor-core products in module `flex`)
# ---------------------------------------------------------------------------------------------
MOE_TILE_ROWS = 32       # pairs per tile of the grouped products on the CUDA cores (moe.cu: MOE_TILE_M)
MOE_TC_TILE_ROWS = 128   # and on the tensor cores (moe_tcgen05.cu: MT_BM)
MOE_TC_MIN_PAIRS = int(os.environ.get("X0NE_MOE_TC_MIN_PAIRS", "1"))     # passes with at least this many (row, choice) pairs take the tensor-core kernel


def moe_max_tiles(pairs: int, experts: int, tile_rows: int = MOE_TILE_ROWS) -> int:
    """Tiles of `tile_rows` pairs a pass of `pairs` (row, choice) pairs over `experts` experts can need at most."""
    full = pairs // tile_rows + experts
    return full if full < pairs else max(pairs, 1)


def moe_tc_takes(dtype: torch.dtype, pairs: int, *widths: int) -> bool:
    """Whether a pass's expert products go to the tensor-core kernel: bfloat16, enough pairs to fill its tiles,
    and every inner width a multiple of 8 (a TMA row of whole 16-byte pieces)."""
    return dtype == torch.bfloat16 and pairs >= MOE_TC_MIN_PAIRS and all(w % 8 == 0 for w in widths)


def moe_route(z: torch.Tensor, correction: torch.Tensor, n: int, groups: int, keep: int, top: int, n_rows: int,
              chosen: torch.Tensor, weights: torch.Tensor, sgate: Optional[torch.Tensor] = None, sg_col: int = 0,
              on_logits: bool = False, sigmoid: bool = False, group_top: int = 1, normalize: bool = False,
              weight_scale: float = 1.0) -> None:
    """The router's choice per row from float32 logits z [rows, >= n] (see moe.cu): `chosen` int32 [rows, top],
    `weights` float32 [rows, top]; `sgate` float32 [rows] = sigmoid(z[:, sg_col]).  `on_logits`: the choice is made on
    z + correction itself (no softmax over all outputs) and the weights are the softmax over the chosen values.
    `sigmoid`: the scores are sigmoid(z) (`correction` may be None).  `group_top`: a group is worth the sum of that many
    of its largest values.  `normalize`: the chosen weights are divided by their sum (+ 1e-20) and multiplied by
    `weight_scale`."""
    lib = _lib("core")
    _need(z, torch.float32, "router logits")
    if correction is not None:
        _need(correction, torch.float32, "router correction")
    elif not sigmoid:
        raise KernelError("moe_route: only a router that scores with the sigmoid goes without a correction")
    _need(chosen, torch.int32, "chosen experts")
    _need(weights, torch.float32, "choice weights")
    if sgate is not None:
        _need(sgate, torch.float32, "shared gate")
    if (correction is not None and correction.numel() != n) or z.numel() < n_rows * z.shape[-1] or chosen.numel() < n_rows * top or weights.numel() < n_rows * top \
            or (sgate is not None and sgate.numel() < n_rows):
        raise KernelError("moe_route: buffers do not match the rows and choices asked for")
    _check(lib, lib.x0ne_moe_route(_ptr(z), z.shape[-1], _ptr(correction), n, groups, keep, top, n_rows, _ptr(chosen),
                                   _ptr(weights), _ptr(sgate), sg_col, 2 if sigmoid else 1 if on_logits else 0, int(group_top),
                                   1 if normalize else 0, float(weight_scale), _stream()), "moe_route")


def moe_group(chosen: torch.Tensor, pairs: int, experts: int, offsets: torch.Tensor, listed: torch.Tensor,
              tiles: torch.Tensor, tile_rows: int = MOE_TILE_ROWS, n_tiles_out: Optional[torch.Tensor] = None) -> None:
    """Lists the pairs expert by expert and fills the table of tiles [max_tiles, 3] (expert, first place, count) for
    tiles of `tile_rows` pairs; `n_tiles_out` (one int32) receives how many tiles exist."""
    lib = _lib("core")
    for t, what in ((chosen, "chosen experts"), (offsets, "expert offsets"), (listed, "listed pairs"), (tiles, "tile table")):
        _need(t, torch.int32, what)
    if chosen.numel() < pairs or listed.numel() < pairs or offsets.numel() < experts + 1:
        raise KernelError("moe_group: buffers smaller than the pairs or experts asked for")
    if n_tiles_out is not None:
        _need(n_tiles_out, torch.int32, "tile count")
    _check(lib, lib.x0ne_moe_group(_ptr(chosen), pairs, experts, _ptr(offsets), _ptr(listed), _ptr(tiles), tiles.numel() // 3,
                                   tile_rows, _ptr(n_tiles_out), _stream()), "moe_group")


def moe_gather_rows(x: torch.Tensor, listed: torch.Tensor, offsets: torch.Tensor, experts: int, top: int, xs: torch.Tensor,
                    pairs: int) -> None:
    """xs[place] = x[listed[place] // top] for every place that holds a pair (bfloat16)."""
    lib = _lib("tc")
    _need(x, torch.bfloat16, "rows")
    _need(xs, torch.bfloat16, "gathered rows")
    if xs.shape[-1] != x.shape[-1] or xs.numel() < pairs * x.shape[-1]:
        raise KernelError("moe_gather_rows: the gathered rows do not match")
    _check(lib, lib.x0ne_moe_gather_rows(_ptr(x), x.shape[-1], _ptr(listed), _ptr(offsets), experts, top, _ptr(xs), pairs,
                                         _stream()), "moe_gather_rows")


def moe_product_tc(which: int, a: torch.Tensor, w: torch.Tensor, listed: torch.Tensor, tiles: torch.Tensor,
                   n_real: torch.Tensor, max_tiles: int, out: torch.Tensor) -> None:
    """The experts' products on tcgen05 over tiles of 128 listed pairs (moe_tcgen05.cu).  which 0: a = the gathered rows
    [places, K], out = relu(.)^2 as bfloat16 [places, N]; which 1: a = those activations, out = float32 [pairs, N] by pair;
    which 2: a as for 0, w [experts, 2 N, K] in blocks of MOE_PAIR_BLOCK gate rows and their up rows, out = silu(gate) * up
    as bfloat16 [places, N]."""
    global tc_used
    lib = _lib("tc")
    _need(a, torch.bfloat16, "expert input")
    _need(w, torch.bfloat16, "expert weights")
    _need(out, torch.float32 if which == 1 else torch.bfloat16, "expert output")
    n_out = w.shape[1] // 2 if which == 2 else w.shape[1]
    if w.dim() != 3 or a.shape[-1] != w.shape[2] or out.shape[-1] != n_out or tiles.numel() < 3 * max_tiles \
            or (which == 2 and w.shape[1] % (2 * MOE_PAIR_BLOCK)):
        raise KernelError("moe_product_tc: shapes do not match")
    tc_used = True
    _check(lib, lib.x0ne_moe_product_tc(which, _ptr(a), a.numel() // a.shape[-1], _ptr(w), w.shape[0], w.shape[1], w.shape[2],
                                        _ptr(listed), _ptr(tiles), _ptr(n_real), max_tiles, _ptr(out),
                                        _ptr(gemm_tc_status(a.device)), _stream()), "moe_product_tc")


MOE_PAIR_BLOCK = 128       # gated experts whose inner width is a multiple of this keep gate and up rows in blocks of it


def moe_product(which: int, a: torch.Tensor, w: torch.Tensor, listed: torch.Tensor, tiles: torch.Tensor, n_tiles: int, top: int,
                out: torch.Tensor, pair_block: int = 0) -> None:
    """The experts' products over the first n_tiles tiles.  which 0: out[pair] = relu(x[pair // top] W_e^T)^2 in the
    activation type; which 1: out[pair] = act[pair] W_e^T in float32.  w is [experts, N, K].  which 2: out[pair] =
    silu(x W_gate_e^T) * (x W_up_e^T) with w [experts, 2 N, K], an expert's gate rows before its up rows, or, with
    `pair_block`, in blocks of that many gate rows followed by the up rows of the same outputs."""
    _need(a, w.dtype, "expert input")
    _need(w, w.dtype, "expert weights")
    _need(out, torch.float32 if which == 1 else w.dtype, "expert output")
    _need(listed, torch.int32, "listed pairs")
    _need(tiles, torch.int32, "tile table")
    n, k = (w.shape[1] // 2 if which == 2 else w.shape[1]), w.shape[2]
    if w.dim() != 3 or a.shape[-1] != k or out.shape[-1] != n or tiles.numel() < 3 * n_tiles or (which == 2 and w.shape[1] % 2):
        raise KernelError("moe_product: shapes do not match")
    if which == 2 and pair_block and n % pair_block:
        raise KernelError(f"moe_product: {n} outputs do not split into blocks of {pair_block}")
    lib = _lib("core")
    _check(lib, lib.x0ne_moe_product(which, _ptr(a), a.shape[-1], _ptr(w), dtype_tag(w.dtype), n, k, _ptr(listed), _ptr(tiles),
                                     n_tiles, top, _ptr(out), int(pair_block) if which == 2 else 0, _stream()), "moe_product")


def moe_combine(y: torch.Tensor, x: torch.Tensor, chosen: torch.Tensor, weights: torch.Tensor, top: int, experts: int,
                shared: Optional[torch.Tensor], sgate: Optional[torch.Tensor], out: torch.Tensor, n_rows: int) -> None:
    """out[row] = sum_j weights[row, j] (y[row * top + j], or x[row] where chosen[row, j] >= experts)
    + sgate[row] * shared[row], in float32."""
    lib = _lib("core")
    _need(y, torch.float32, "expert outputs")
    _need(x, x.dtype, "rows")
    _need(out, x.dtype, "feed-forward output")
    hidden = x.shape[-1]
    if y.shape[-1] != hidden or out.shape[-1] != hidden or y.numel() < n_rows * top * hidden or out.numel() < n_rows * hidden:
        raise KernelError("moe_combine: widths or rows do not match")
    if shared is not None:
        _need(shared, x.dtype, "shared expert output")
    _check(lib, lib.x0ne_moe_combine(_ptr(y), _ptr(x), dtype_tag(x.dtype), _ptr(chosen), _ptr(weights), top, experts,
                                     _ptr(shared), _ptr(sgate), _ptr(out), n_rows, hidden, _stream()), "moe_combine")


def qk_norm_rope_kv_write(qkv: torch.Tensor, q_norm: Optional[torch.Tensor], k_norm: Optional[torch.Tensor],
                          inv_freq: Optional[torch.Tensor], rotary_dim: int, q_out: torch.Tensor,
                          cache: PagedCacheArg, row_slot: torch.Tensor, row_pos: torch.Tensor, n_rows: int,
                          q_heads: int, eps: float, write_kv: bool = True,
                          rope_table: Optional[torch.Tensor] = None) -> None:
    """q/k head norm, rotation and cache write.  `rope_table` (float32 [positions, rotary_dim]: each
    row the cosines then the sines of position * inv_freq) replaces the on-the-fly sines and cosines
    for the positions it covers."""
    lib = _lib("core")
    _need(qkv, qkv.dtype, "qkv")
    _need(q_out, qkv.dtype, "q output")
    _need(row_slot, torch.int32, "row slots")
    _need(row_pos, torch.int32, "row positions")
    hd, kvh = cache.head_dim, cache.kv_heads
    if qkv.shape[-1] != (q_heads + 2 * kvh) * hd or q_out.shape[-1] != q_heads * hd:
        raise KernelError("rope: qkv or q widths do not match the head counts")
    if qkv.numel() < n_rows * qkv.shape[-1] or q_out.numel() < n_rows * q_out.shape[-1]:
        raise KernelError("rope: buffers smaller than the rows asked for")
    for w, what in ((q_norm, "q_norm"), (k_norm, "k_norm")):
        if w is not None:
            _need(w, torch.float32, what)
            if w.numel() != hd:
                raise KernelError(f"rope: {what} has {w.numel()} values, head_dim is {hd}")
    if inv_freq is not None:
        _need(inv_freq, torch.float32, "inv_freq")
        if inv_freq.numel() * 2 != rotary_dim:
            raise KernelError("rope: inv_freq length is not rotary_dim / 2")
    table_positions = 0
    if rope_table is not None:
        _need(rope_table, torch.float32, "rope table")
        if rope_table.dim() != 2 or rope_table.shape[1] != rotary_dim:
            raise KernelError("rope: the table is not [positions, rotary_dim]")
        table_positions = rope_table.shape[0]
    _check(lib, lib.x0ne_qk_norm_rope_kv_write(
        _ptr(qkv), dtype_tag(qkv.dtype), _ptr(q_norm), _ptr(k_norm), _ptr(inv_freq), rotary_dim,
        _ptr(q_out), cache, _ptr(row_slot), _ptr(row_pos), n_rows, q_heads, eps,
        1 if write_kv else 0, _ptr(rope_table), table_positions, _stream()), "qk_norm_rope_kv_write")


def attention_rows(q: torch.Tensor, out: torch.Tensor, cache: PagedCacheArg, row_slot: torch.Tensor,
                   row_pos: torch.Tensor, n_rows: int, q_heads: int, scale: float, window: int = 0,
                   extra: Optional[AttnExtraArg] = None) -> None:
    """The plain attention kernel: keys up to 2,048 wide, values up to 512, any window (0 = none), and
    what `extra` asks for (see `attn_extra`).  With `extra.q_ld` the queries are rows of a wider buffer."""
    lib = _lib("core")
    _need(out, torch.float32 if extra is not None and extra.out_f32 else q.dtype, "attention output")
    _need(row_slot, torch.int32, "row slots")
    _need(row_pos, torch.int32, "row positions")
    if not q.is_cuda or (extra is None or not extra.q_ld) and not q.is_contiguous():
        raise KernelError("attention: q is not a contiguous GPU tensor")
    vd = extra.v_from_k if extra is not None and extra.v_from_k else cache.value_dim
    width, out_width = q_heads * cache.head_dim, q_heads * vd
    if extra is None or not extra.q_ld:
        if q.shape[-1] != width or q.numel() < n_rows * width:
            raise KernelError("attention: q does not match the head counts and rows")
    if out.shape[-1] != out_width or out.numel() < n_rows * out_width:
        raise KernelError("attention: the output does not match the head counts and rows")
    if extra is None:
        _check(lib, lib.x0ne_attention_rows(_ptr(q), _ptr(out), dtype_tag(q.dtype), cache, _ptr(row_slot),
                                            _ptr(row_pos), n_rows, q_heads, scale, window,
                                            _stream()), "attention_rows")
    else:
        _check(lib, lib.x0ne_attention_rows_ex(_ptr(q), _ptr(out), dtype_tag(q.dtype), cache, _ptr(row_slot),
                                               _ptr(row_pos), n_rows, q_heads, scale, window, extra,
                                               _stream()), "attention_rows")


def glu_clipped(gate_up: torch.Tensor, out: torch.Tensor, n_rows: int, limit: float, slope: float, shift: float) -> None:
    """out = g sigmoid(slope g) (u + shift) with g = min(gate, limit), u = clamp(up, -limit, limit), on the
    packed [gate; up] rows."""
    lib = _lib("core")
    _need(gate_up, gate_up.dtype, "gate_up")
    _need(out, gate_up.dtype, "activation output")
    inter = out.shape[-1]
    if gate_up.shape[-1] != 2 * inter or gate_up.numel() < n_rows * 2 * inter or out.numel() < n_rows * inter:
        raise KernelError("glu_clipped: widths or rows do not match")
    _check(lib, lib.x0ne_glu_clipped(_ptr(gate_up), _ptr(out), dtype_tag(out.dtype), n_rows, inter, limit, slope, shift,
                                     _stream()), "glu_clipped")


def kv_write_blend(src: torch.Tensor, k_col: int, v_col: int, cache: PagedCacheArg, row_slot: torch.Tensor,
                   row_pos: torch.Tensor, n_rows: int, mode: int = 0, v_first: Optional[torch.Tensor] = None,
                   blend: Optional[torch.Tensor] = None) -> None:
    """Writes the keys (columns from k_col) and values (from v_col) of `src` rows into the cache.  mode 1
    also keeps the values in `v_first`; mode 2 writes (1 - blend) v + blend v_first, `blend` one float32
    on the device."""
    lib = _lib("core")
    _need(src, src.dtype, "projection rows")
    _need(row_slot, torch.int32, "row slots")
    _need(row_pos, torch.int32, "row positions")
    if src.numel() < n_rows * src.shape[-1] or row_slot.numel() < n_rows or row_pos.numel() < n_rows:
        raise KernelError("kv_write: buffers smaller than the rows asked for")
    if v_first is not None:
        _need(v_first, src.dtype, "first values")
        if v_first.shape[-1] != cache.kv_heads * cache.value_dim or v_first.numel() < n_rows * v_first.shape[-1]:
            raise KernelError("kv_write: the buffer of first values does not match the cache's values")
    if blend is not None:
        _need(blend, torch.float32, "blend weight")
    _check(lib, lib.x0ne_kv_write_blend(_ptr(src), dtype_tag(src.dtype), src.shape[-1], k_col, v_col, _ptr(v_first),
                                        _ptr(blend), mode, cache, _ptr(row_slot), _ptr(row_pos), n_rows, _stream()),
           "kv_write_blend")


def latent_prepare(src: torch.Tensor, dkv_col: int, q_abs: torch.Tensor, norm_w: torch.Tensor, eps: float,
                   freq: Optional[torch.Tensor], mag: float, table: Optional[torch.Tensor], q_out: torch.Tensor, heads: int,
                   dim: int, rot: int, rank: int, cache: PagedCacheArg, row_slot: torch.Tensor, row_pos: torch.Tensor,
                   n_rows: int, write_cache: bool = True) -> None:
    """Latent attention's rows: normed latent and rotated shared key part into the cache, and the queries
    [q_abs | rotated part] per head (see mixer_rows.cu).  `q_abs` is [heads, rows, rank]."""
    lib = _lib("core")
    _need(src, src.dtype, "projection rows")
    _need(q_abs, src.dtype, "queries in latent space")
    _need(q_out, src.dtype, "query output")
    _need(norm_w, torch.float32, "latent norm weight")
    _need(row_slot, torch.int32, "row slots")
    _need(row_pos, torch.int32, "row positions")
    if q_abs.dim() != 3 or q_abs.shape[0] != heads or q_abs.shape[2] != rank or q_abs.shape[1] < n_rows:
        raise KernelError("latent_prepare: q_abs is not [heads, rows, rank]")
    if norm_w.numel() != rank or q_out.shape[-1] != heads * (rank + rot) or q_out.numel() < n_rows * q_out.shape[-1] \
            or src.numel() < n_rows * src.shape[-1]:
        raise KernelError("latent_prepare: widths or rows do not match")
    positions = 0
    if rot:
        _need(freq, torch.float32, "rotary frequencies")
        if freq.numel() * 2 != rot:
            raise KernelError("latent_prepare: frequencies are not rot / 2")
        if table is not None:
            _need(table, torch.float32, "rotary table")
            if table.dim() != 2 or table.shape[1] != rot:
                raise KernelError("latent_prepare: the table is not [positions, rot]")
            positions = table.shape[0]
    _check(lib, lib.x0ne_latent_prepare(_ptr(src), dtype_tag(src.dtype), src.shape[-1], dkv_col, _ptr(q_abs),
                                        q_abs.stride(0), _ptr(norm_w), eps, _ptr(freq), mag, _ptr(table), positions,
                                        _ptr(q_out), heads, dim, rot, rank, cache, _ptr(row_slot), _ptr(row_pos), n_rows,
                                        1 if write_cache else 0, _stream()), "latent_prepare")


def batched_product(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[b] = a[b] @ w[b]^T for a [B, M, K], w [B, N, K], out [B, M, N]; `a` and `out` may be strided
    views (last axis contiguous), `w` is contiguous.  float32: this library's fixed-order FMA kernel, one
    product per z of the grid; bfloat16: the vendor's strided batched product (float32 accumulation)."""
    if a.dim() != 3 or w.dim() != 3 or out.dim() != 3 or a.shape[0] != w.shape[0] or a.shape[2] != w.shape[2] \
            or out.shape != (a.shape[0], a.shape[1], w.shape[1]) or a.stride(2) != 1 or out.stride(2) != 1 or not w.is_contiguous():
        raise KernelError(f"batched_product: shapes a {tuple(a.shape)} w {tuple(w.shape)} out {tuple(out.shape)}")
    b, m, k = a.shape
    n = w.shape[1]
    if m == 0:
        return
    if a.dtype == torch.float32:
        lib = _lib("core")
        _check(lib, lib.x0ne_gemm_f32_nt_batched(_ptr(a), _ptr(w), _ptr(out), m, n, k, a.stride(1), k, out.stride(1), b,
                                                 a.stride(0), n * k, out.stride(0), _stream()), "gemm_f32_nt_batched")
    elif a.dtype == torch.bfloat16:
        if out.is_contiguous():
            torch.bmm(a, w.transpose(1, 2), out=out)
        else:
            out.copy_(torch.bmm(a, w.transpose(1, 2)))
    else:
        raise KernelError(f"batched_product: no product for {a.dtype}")


# ---------------------------------------------------------------------------------------------
# bfloat16 attention for free key / value widths, masks, sinks and gates (module `flex`)
# ---------------------------------------------------------------------------------------------
PREFILL_TILE_ROWS = 128      # rows of a tile of every bfloat16 prefill attention kernel (the pass tables are built with it)
FLEX_SMEM_LIMIT = 200 * 1024


FLEX_VALUE_BUCKETS = (16, 32, 48, 64, 96, 128, 192, 256)     # the value widths the kernels are compiled for


def flex_value_bucket(vd: int) -> int:
    return next((b for b in FLEX_VALUE_BUCKETS if vd <= b), 0)


def attention_flex_takes(cache: PagedCacheArg, dtype: torch.dtype, v_from_k: int = 0, decode: bool = False) -> bool:
    """Whether the general bfloat16 attention kernels take this shape; else the plain kernel does."""
    if dtype != torch.bfloat16 or cache.page_size != 64:
        return False
    vd = v_from_k or cache.value_dim
    dkp, vdp = -(-cache.head_dim // 16) * 16, flex_value_bucket(vd)
    if vd <= 0 or vdp == 0:
        return False
    ks = (max(dkp, vdp) if v_from_k else dkp) + 8
    stage = (64 * ks + (0 if v_from_k else 64 * (vdp + 8))) * 2        # a key tile and a value tile
    tiles = 2 * stage
    if decode:
        smem = 16 * ks * 2 + max(2 * stage, 4 * 16 * (vdp + 2) * 4)
    else:
        smem = 128 * ks * 2 + tiles
    return smem <= FLEX_SMEM_LIMIT


def attention_flex_prefill(q: torch.Tensor, out: torch.Tensor, cache: PagedCacheArg, tile_seq: torch.Tensor,
                           tile_row0: torch.Tensor, n_tiles: int, seq_first_row: torch.Tensor, seq_slot: torch.Tensor,
                           seq_pos0: torch.Tensor, q_heads: int, scale: float, window: int, extra: AttnExtraArg) -> None:
    """Flash attention of a pass whose sequences bring several rows; tiles of up to 128 rows of one sequence."""
    lib = _lib("flex")
    _need(out, torch.float32 if extra.out_f32 else torch.bfloat16, "attention output")
    if q.dtype != torch.bfloat16 or not q.is_cuda:
        raise KernelError("attention_flex: q is not a bfloat16 GPU tensor")
    for t, what in ((tile_seq, "tile sequences"), (tile_row0, "tile rows"), (seq_first_row, "sequence rows"),
                    (seq_slot, "sequence slots"), (seq_pos0, "sequence positions")):
        _need(t, torch.int32, what)
    if tile_seq.numel() < n_tiles or tile_row0.numel() < n_tiles:
        raise KernelError("attention_flex: tile tables shorter than the tiles asked for")
    vd = extra.v_from_k or cache.value_dim
    if out.shape[-1] != q_heads * vd:
        raise KernelError("attention_flex: the output width does not match the head counts")
    for first in range(0, n_tiles, 65535):
        n = min(65535, n_tiles - first)
        _check(lib, lib.x0ne_attention_flex_prefill(
            _ptr(q), _ptr(out), cache, tile_seq.data_ptr() + 4 * first, tile_row0.data_ptr() + 4 * first, n,
            _ptr(seq_first_row), _ptr(seq_slot), _ptr(seq_pos0), q_heads, scale, window, extra, _stream()),
            "attention_flex_prefill")


def attention_flex_scratch_bytes(n_rows: int, q_heads: int, kv_heads: int, vd: int, splits: int) -> int:
    chunks, vdp = -(-(q_heads // kv_heads) // 16), flex_value_bucket(vd)
    return n_rows * kv_heads * chunks * splits * 16 * (vdp + 2) * 4 if splits > 1 else 0


def attention_flex_decode(q: torch.Tensor, out: torch.Tensor, cache: PagedCacheArg, row_slot: torch.Tensor,
                          row_pos: torch.Tensor, n_rows: int, q_heads: int, scale: float, window: int,
                          extra: AttnExtraArg, splits: int = 1, scratch: Optional[torch.Tensor] = None) -> None:
    """One query row per sequence; `splits` blocks share a row's pages and meet in `scratch`."""
    lib = _lib("flex")
    _need(out, torch.float32 if extra.out_f32 else torch.bfloat16, "attention output")
    if q.dtype != torch.bfloat16 or not q.is_cuda:
        raise KernelError("attention_flex: q is not a bfloat16 GPU tensor")
    _need(row_slot, torch.int32, "row slots")
    _need(row_pos, torch.int32, "row positions")
    vd = extra.v_from_k or cache.value_dim
    if out.shape[-1] != q_heads * vd or out.numel() < n_rows * q_heads * vd or row_slot.numel() < n_rows or row_pos.numel() < n_rows:
        raise KernelError("attention_flex: output or row tables do not match the rows asked for")
    nbytes = scratch.numel() * scratch.element_size() if scratch is not None else 0
    _check(lib, lib.x0ne_attention_flex_decode(_ptr(q), _ptr(out), cache, _ptr(row_slot), _ptr(row_pos), n_rows, q_heads,
                                               scale, window, extra, splits, _ptr(scratch), nbytes, _stream()),
           "attention_flex_decode")
    if splits > 1:
        global LAUNCHES
        LAUNCHES += 1


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, n_rows: int) -> None:
    lib = _lib("core")
    _need(gate_up, gate_up.dtype, "gate_up")
    _need(out, gate_up.dtype, "swiglu output")
    inter = out.shape[-1]
    if gate_up.shape[-1] != 2 * inter or gate_up.numel() < n_rows * 2 * inter or out.numel() < n_rows * inter:
        raise KernelError("swiglu: widths or rows do not match")
    _check(lib, lib.x0ne_swiglu(_ptr(gate_up), _ptr(out), dtype_tag(out.dtype), n_rows, inter,
                                _stream()), "swiglu")


def gemm_f32_nt(a: torch.Tensor, w: torch.Tensor, c: torch.Tensor, m: int) -> None:
    """c[:m] = a[:m] @ w.T in true float32, one fixed-order FMA chain per output."""
    lib = _lib("core")
    _need(a, torch.float32, "gemm input")
    _need(w, torch.float32, "gemm weight")
    _need(c, torch.float32, "gemm output")
    n, k = w.shape
    if a.shape[-1] != k or c.shape[-1] != n or a.numel() < m * k or c.numel() < m * n:
        raise KernelError(f"gemm_f32: shapes a {tuple(a.shape)} w {tuple(w.shape)} c {tuple(c.shape)} m {m}")
    _check(lib, lib.x0ne_gemm_f32_nt(_ptr(a), _ptr(w), _ptr(c), m, n, k, k, k,
                                     n, _stream()), "gemm_f32_nt")


def sample(logits: torch.Tensor, n_rows: int, out_token: torch.Tensor, *, temperature=None, top_p=None, seed=None,
           draw_counter=None, stop_ids=None, finished=None, budget=None, next_token=None, next_pos=None,
           status=None, row_best=None) -> None:
    """Picks a token per logits row on the device (see sampling.cu for the rules).  `stop_ids` may
    be padded with -1 (no token has that id).  With `status` (one int32 on the device) the kernel
    also copies that int to out_token[n_rows], so it reaches the host with the picks.  With
    `row_best` (one int64 per row, zero; left zero) a launch of many blocks per row finds the rows'
    largest logits first, which one block per row takes 17 us for at a vocabulary of 151,936."""
    lib = _lib("core")
    _need(logits, torch.float32, "logits")
    _need(out_token, torch.int32, "token output")
    if logits.dim() != 2 or logits.shape[0] < n_rows or out_token.numel() < n_rows:
        raise KernelError("sample: logits or output smaller than the rows asked for")
    for t, dt, what in ((temperature, torch.float32, "temperature"), (top_p, torch.float32, "top_p"),
                        (seed, torch.int64, "seed"), (draw_counter, torch.int32, "draw counter"),
                        (finished, torch.int32, "finished flags"), (budget, torch.int32, "budget"),
                        (next_token, torch.int32, "next token"), (next_pos, torch.int32, "next position")):
        if t is not None:
            _need(t, dt, what)
            if t.numel() < n_rows:
                raise KernelError(f"sample: {what} shorter than the rows asked for")
    if status is not None:
        _need(status, torch.int32, "status word")
        if out_token.numel() < n_rows + 1:
            raise KernelError("sample: no room for the status word after the picks")
    if row_best is not None:
        _need(row_best, torch.int64, "largest-logit scratch")
        if row_best.numel() < n_rows:
            raise KernelError("sample: largest-logit scratch shorter than the rows asked for")
    n_stop = 0
    if stop_ids is not None and stop_ids.numel() > 0:
        _need(stop_ids, torch.int32, "stop ids")
        n_stop = stop_ids.numel()
    io = SampleIOArg(_ptr(logits), _ptr(temperature), _ptr(top_p), _ptr(seed), _ptr(draw_counter),
                     _ptr(stop_ids if n_stop else None), _ptr(finished), _ptr(budget), _ptr(out_token),
                     _ptr(next_token), _ptr(next_pos), _ptr(status), _ptr(row_best), logits.stride(0), logits.shape[1], n_stop)
    _check(lib, lib.x0ne_sample(io, n_rows, _stream()), "sample")
    if row_best is not None and n_rows > 0:
        global LAUNCHES
        LAUNCHES += 1        # that entry point launched two kernels


# ---------------------------------------------------------------------------------------------
# bfloat16 tensor-core attention (module `fast`)
# ---------------------------------------------------------------------------------------------
def fast_attention_takes(cache: PagedCacheArg, dtype: torch.dtype) -> bool:
    """Whether the tensor-core attention kernels take this shape; otherwise the plain kernel does."""
    return dtype == torch.bfloat16 and cache.page_size == 64 and cache.head_dim % 16 == 0 \
        and 16 <= cache.head_dim <= 128 and cache.v_dim == 0


def attention_prefill_bf16(q: torch.Tensor, out: torch.Tensor, cache: PagedCacheArg, tile_seq: torch.Tensor,
                           tile_row0: torch.Tensor, n_tiles: int, seq_first_row: torch.Tensor,
                           seq_slot: torch.Tensor, seq_pos0: torch.Tensor, q_heads: int, scale: float,
                           window: int = 0) -> None:
    """Causal flash attention of a pass whose sequences bring several rows; a tile is up to
    `attention_prefill_tile_rows()` consecutive rows of one sequence."""
    lib = _lib("fast")
    _need(q, torch.bfloat16, "q")
    _need(out, torch.bfloat16, "attention output")
    for t, what in ((tile_seq, "tile sequences"), (tile_row0, "tile rows"), (seq_first_row, "sequence rows"),
                    (seq_slot, "sequence slots"), (seq_pos0, "sequence positions")):
        _need(t, torch.int32, what)
    if tile_seq.numel() < n_tiles or tile_row0.numel() < n_tiles:
        raise KernelError("attention_prefill: tile tables shorter than the tiles asked for")
    if q.shape[-1] != q_heads * cache.head_dim or out.shape[-1] != q.shape[-1]:
        raise KernelError("attention_prefill: q or output width does not match the head counts")
    for first in range(0, n_tiles, 65535):
        n = min(65535, n_tiles - first)
        _check(lib, lib.x0ne_attention_prefill_bf16(
            _ptr(q), _ptr(out), cache, tile_seq.data_ptr() + 4 * first,
            tile_row0.data_ptr() + 4 * first, n, _ptr(seq_first_row), _ptr(seq_slot), _ptr(seq_pos0),
            q_heads, scale, window, _stream()), "attention_prefill_bf16")


def attention_prefill_tile_rows() -> int:
    """Rows of one tile of the prefill attention kernel (callers build their tile tables with it)."""
    return int(_lib("fast").x0ne_attention_prefill_tile_rows())


def attention_decode_blocks_per_sm() -> int:
    return int(_lib("fast").x0ne_attention_decode_blocks_per_sm())


_max_clusters = {}


def attention_decode_max_clusters(head_dim: int, splits: int) -> int:
    """Clusters of `splits` blocks of the decode kernel that run at once on this GPU (0: unknown)."""
    key = (torch.cuda.current_device(), head_dim, splits)
    if key not in _max_clusters:
        _max_clusters[key] = int(_lib("fast").x0ne_attention_decode_max_clusters(c_int(head_dim), c_int(splits)))
    return _max_clusters[key]


def attention_decode_scratch_bytes(n_rows: int, q_heads: int, kv_heads: int, head_dim: int, splits: int) -> int:
    lib = _lib("fast")
    lib.x0ne_attention_decode_scratch_bytes.restype = c_int64
    return int(lib.x0ne_attention_decode_scratch_bytes(c_int(n_rows), c_int(q_heads), c_int(kv_heads),
                                                       c_int(head_dim), c_int(splits)))


ATTENTION_DECODE_CLUSTER_SPLITS = 8     # splits that can merge inside one thread-block cluster
ATTENTION_DECODE_MAX_SPLITS = 64        # blocks per (sequence, kv head) the kernel takes


def attention_decode_bf16(q: torch.Tensor, out: torch.Tensor, cache: PagedCacheArg, row_slot: torch.Tensor,
                          row_pos: torch.Tensor, n_rows: int, q_heads: int, scale: float, window: int, splits: int,
                          scratch: Optional[torch.Tensor], groups: int = 1) -> None:
    """Split-KV flash decoding: one query row per sequence.  `scratch` (uint8, zero when first
    used; the kernel leaves its counters at zero) holds the partial results when splits > 1; without
    it (and with at most 8 splits) the splits merge inside a thread-block cluster instead.  With
    `groups` > 1 the splits are `groups` clusters of splits / groups blocks (2 to 8): each cluster
    merges in shared memory and the clusters' results meet in `scratch` (sized for `groups` parts)."""
    lib = _lib("fast")
    _need(q, torch.bfloat16, "q")
    _need(out, torch.bfloat16, "attention output")
    _need(row_slot, torch.int32, "row slots")
    _need(row_pos, torch.int32, "row positions")
    width = q_heads * cache.head_dim
    if q.shape[-1] != width or out.shape[-1] != width or q.numel() < n_rows * width or out.numel() < n_rows * width:
        raise KernelError("attention_decode: q or output do not match the head counts and rows")
    if row_slot.numel() < n_rows or row_pos.numel() < n_rows:
        raise KernelError("attention_decode: row tables shorter than the rows asked for")
    nbytes = 0
    if scratch is not None:
        _need(scratch, torch.uint8, "decode scratch")
        nbytes = scratch.numel()
    if groups > 1:
        _check(lib, lib.x0ne_attention_decode_grouped_bf16(
            _ptr(q), _ptr(out), cache, _ptr(row_slot), _ptr(row_pos), n_rows, q_heads, scale,
            window, splits, groups, _ptr(scratch), nbytes, _stream()), "attention_decode_grouped_bf16")
        return
    _check(lib, lib.x0ne_attention_decode_bf16(
        _ptr(q), _ptr(out), cache, _ptr(row_slot), _ptr(row_pos), n_rows, q_heads, scale,
        window, splits, _ptr(scratch), nbytes, _stream()), "attention_decode_bf16")


# ---------------------------------------------------------------------------------------------
# bfloat16 small-M weight-streaming product (module `fast`)
# ---------------------------------------------------------------------------------------------
SMALL_M_MAX_ROWS = 32       # rows the weight-streaming kernel takes (which products use it: routes.py)
_sm_count = {}


def _sms(device) -> int:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    n = _sm_count.get(idx)
    if n is None:
        n = _sm_count[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return n


def gemm_smallm_takes(w: torch.Tensor, m: int, swiglu: bool = False) -> bool:
    """Whether the weight-streaming kernel takes this shape."""
    return w.dtype == torch.bfloat16 and 0 < m <= SMALL_M_MAX_ROWS and w.shape[1] % 8 == 0 and not (swiglu and w.shape[0] % 2)


def gemm_bf16_smallm(x: torch.Tensor, w: torch.Tensor, y: torch.Tensor, m: int, swiglu: bool = False,
                     glu: Optional[tuple] = None) -> None:
    """y[:m] = x[:m] @ w.T for m <= 32 by streaming w once; y is bfloat16 or float32.  With
    `swiglu`, w is the packed [gate; up] weight and y[:m] = silu(x gate^T) * (x up^T); with `glu` =
    (limit, slope, shift) besides, the clipped unit min(g, limit) sigmoid(slope g) (clamp(u) + shift)."""
    lib = _lib("fast")
    _need(x, torch.bfloat16, "gemm input")
    _need(w, torch.bfloat16, "gemm weight")
    _need(y, y.dtype, "gemm output")
    rows, k = w.shape
    n = rows // 2 if swiglu else rows
    if x.shape[-1] != k or y.shape[-1] != n or x.numel() < m * k or y.numel() < m * n or (swiglu and rows % 2):
        raise KernelError(f"gemm_smallm: shapes x {tuple(x.shape)} w {tuple(w.shape)} y {tuple(y.shape)} m {m}")
    if y.dtype == torch.float32 and not swiglu:
        kind = 1
    elif y.dtype == torch.bfloat16:
        kind = 2 if swiglu else 0
    else:
        raise KernelError(f"gemm_smallm: no output kind for {y.dtype} (swiglu={swiglu})")
    if glu is not None and swiglu:
        _check(lib, lib.x0ne_gemm_bf16_smallm_glu(_ptr(w), _ptr(x), _ptr(y), m, n, k, n, kind, _sms(w.device),
                                                  glu[0], glu[1], glu[2], _stream()), "gemm_bf16_smallm")
        return
    _check(lib, lib.x0ne_gemm_bf16_smallm(_ptr(w), _ptr(x), _ptr(y), m, n, k, n,
                                          kind, _sms(w.device), _stream()), "gemm_bf16_smallm")


# ---------------------------------------------------------------------------------------------
# bfloat16 product on tcgen05 tensor cores with TMA operands (module `tc`), for passes with many rows
# ---------------------------------------------------------------------------------------------
_tc_status = {}
tc_used = False          # set when a tcgen05 product was launched since the last check_tc_status()


def gemm_tc_takes(w: torch.Tensor, m: int) -> bool:
    """Whether the tcgen05 product for many rows takes this shape (from which row count it is used: routes.py)."""
    return w.dtype == torch.bfloat16 and m >= 1 and w.shape[1] % 8 == 0


def check_tc_status(device) -> None:
    """Raises if a tcgen05 kernel reported a barrier wait that ran out (reads one int back)."""
    global tc_used
    if not tc_used:
        return
    tc_used = False
    st = int(gemm_tc_status(device)[0])
    if st != 0:
        gemm_tc_status(device).zero_()
        raise KernelError(describe_tc_status(st))


def describe_tc_status(st: int) -> str:
    """The message for a status word that is not zero: one bit per kind of wait that ran out."""
    codes = [b for b in range(32) if st >> b & 1]
    return (f"a tcgen05 kernel gave up waiting on a barrier (codes {codes}; products: 1 copy, 2 MMA, "
            "3 epilogue, 4 accumulator; attention: 5 queries, 6 keys, 13 and 15 values, 7 probabilities, "
            "8, 11 and 14 output, 10, 12 and 17 scores, 16 and 18 the other half of the row; 9: misaligned "
            "shared memory); its output is not valid")


def gemm_tc_status(device) -> torch.Tensor:
    """The int the tcgen05 kernels report a timed-out barrier wait in (0 = all waits succeeded)."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _tc_status.get(idx)
    if t is None:
        t = _tc_status[idx] = torch.zeros(1, dtype=torch.int32, device=device)
    return t


def gemm_bf16_tcgen05(x: torch.Tensor, w: torch.Tensor, y: torch.Tensor, m: int, swiglu: bool = False,
                      pair: bool = True, glu: Optional[tuple] = None) -> None:
    """y[:m] = x[:m] @ w.T on the tcgen05 tensor cores (128 x 256 tiles, TMA loads, accumulator in
    tensor memory; with `pair`, pairs of blocks on 256 x 256 tiles); y is bfloat16 or float32.  With `swiglu`, w is the packed [gate; up] weight and
    y[:m] = silu(x gate^T) * (x up^T).  Needs K % 8 == 0."""
    lib = _lib("tc")
    _need(x, torch.bfloat16, "gemm input")
    _need(w, torch.bfloat16, "gemm weight")
    _need(y, y.dtype, "gemm output")
    rows, k = w.shape
    n = rows // 2 if swiglu else rows
    if x.shape[-1] != k or y.shape[-1] != n or x.numel() < m * k or y.numel() < m * n or (swiglu and rows % 2):
        raise KernelError(f"gemm_tc: shapes x {tuple(x.shape)} w {tuple(w.shape)} y {tuple(y.shape)} m {m}")
    if y.dtype == torch.float32 and not swiglu:
        kind = 1
    elif y.dtype == torch.bfloat16:
        kind = 2 if swiglu else 0
    else:
        raise KernelError(f"gemm_tc: no output kind for {y.dtype} (swiglu={swiglu})")
    global tc_used
    tc_used = True
    if glu is not None and swiglu:       # (limit, slope, shift): the clipped gated unit instead of SwiGLU
        _check(lib, lib.x0ne_gemm_bf16_tcgen05_glu(_ptr(w), _ptr(x), _ptr(y), m, n, k, n, kind, 1 if pair else 0,
                                                   _ptr(gemm_tc_status(w.device)), glu[0], glu[1], glu[2], _stream()),
               "gemm_bf16_tcgen05")
        return
    _check(lib, lib.x0ne_gemm_bf16_tcgen05(_ptr(w), _ptr(x), _ptr(y), m, n, k, n,
                                           kind, 1 if pair else 0, _ptr(gemm_tc_status(w.device)),
                                           _stream()), "gemm_bf16_tcgen05")


SKINNY_MIN_ROWS, SKINNY_MAX_ROWS = 9, 64


def gemm_skinny_tc_takes(w: torch.Tensor, m: int) -> bool:
    """Whether the tcgen05 product for few rows takes this shape (more rows than the weight-streaming
    kernel is best at, few enough for one accumulator tile)."""
    return w.dtype == torch.bfloat16 and SKINNY_MIN_ROWS <= m <= SKINNY_MAX_ROWS and w.shape[1] % 8 == 0


def product_kernel(w: torch.Tensor, m: int, fused: bool = False) -> str:
    """The kernel the routing table names for m rows against w, or "library" where that kernel does not
    take the shape (a width that is no multiple of 8)."""
    from . import routes
    kernel = routes.kernel_for(m, w.shape[0], w.shape[1], fused=fused, sms=_sms(w.device))
    can = {"smallm": gemm_smallm_takes(w, m, fused), "skinny": gemm_skinny_tc_takes(w, m), "tc_pair": gemm_tc_takes(w, m),
           "library": True}[kernel]
    return kernel if can else "library"


def gemm_bf16_skinny_tcgen05(x: torch.Tensor, w: torch.Tensor, y: torch.Tensor, m: int, swiglu: bool = False,
                             glu: Optional[tuple] = None) -> None:
    """y[:m] = x[:m] @ w.T for up to 64 rows on tcgen05, K cut over the blocks of a cluster that add
    their partial sums through shared memory; y is bfloat16 or float32.  With `swiglu`, w is the
    packed [gate; up] weight and y[:m] = silu(x gate^T) * (x up^T).  Failures of its bounded waits
    show in `gemm_tc_status`."""
    global tc_used
    lib = _lib("tc")
    _need(x, torch.bfloat16, "gemm input")
    _need(w, torch.bfloat16, "gemm weight")
    _need(y, y.dtype, "gemm output")
    rows, k = w.shape
    n = rows // 2 if swiglu else rows
    if x.shape[-1] != k or y.shape[-1] != n or x.numel() < m * k or y.numel() < m * n or (swiglu and rows % 2):
        raise KernelError(f"gemm_skinny_tc: shapes x {tuple(x.shape)} w {tuple(w.shape)} y {tuple(y.shape)} m {m}")
    if y.dtype == torch.float32 and not swiglu:
        kind = 1
    elif y.dtype == torch.bfloat16:
        kind = 2 if swiglu else 0
    else:
        raise KernelError(f"gemm_skinny_tc: no output kind for {y.dtype} (swiglu={swiglu})")
    tc_used = True
    x_rows = x.numel() // k      # rows really behind x: the copies may read them all (their results are not used)
    if glu is not None and swiglu:       # (limit, slope, shift): the clipped gated unit instead of SwiGLU
        _check(lib, lib.x0ne_gemm_bf16_skinny_tcgen05_glu(_ptr(w), _ptr(x), x_rows, _ptr(y), m, n, k, n, kind,
                                                          _ptr(gemm_tc_status(x.device)), glu[0], glu[1], glu[2], _stream()),
               "gemm_bf16_skinny_tcgen05")
        return
    _check(lib, lib.x0ne_gemm_bf16_skinny_tcgen05(_ptr(w), _ptr(x), x_rows, _ptr(y), m, n, k, n, kind,
                                                  _ptr(gemm_tc_status(x.device)), _stream()), "gemm_bf16_skinny_tcgen05")


def attention_tc_takes(cache: PagedCacheArg, dtype: torch.dtype) -> bool:
    """Whether the tcgen05 prefill attention takes this shape."""
    return dtype == torch.bfloat16 and cache.page_size == 64 and cache.head_dim in (64, 128) and cache.v_dim == 0


def attention_prefill_tcgen05(q: torch.Tensor, out: torch.Tensor, cache: PagedCacheArg, tile_seq: torch.Tensor,
                              tile_row0: torch.Tensor, n_tiles: int, seq_first_row: torch.Tensor,
                              seq_slot: torch.Tensor, seq_pos0: torch.Tensor, q_heads: int, scale: float,
                              window: int = 0) -> None:
    """Causal flash attention of a pass whose sequences bring several rows, on tcgen05 with TMA loads;
    tiles are up to 128 consecutive rows of one sequence (`attention_prefill_tile_rows()`)."""
    global tc_used
    lib = _lib("tc")
    _need(q, torch.bfloat16, "q")
    _need(out, torch.bfloat16, "attention output")
    for t, what in ((tile_seq, "tile sequences"), (tile_row0, "tile rows"), (seq_first_row, "sequence rows"),
                    (seq_slot, "sequence slots"), (seq_pos0, "sequence positions")):
        _need(t, torch.int32, what)
    if tile_seq.numel() < n_tiles or tile_row0.numel() < n_tiles:
        raise KernelError("attention_prefill_tc: tile tables shorter than the tiles asked for")
    if q.dim() != 2 or q.shape[-1] != q_heads * cache.head_dim or out.shape != q.shape:
        raise KernelError("attention_prefill_tc: q or output do not match the head counts")
    tc_used = True
    for first in range(0, n_tiles, 65535):
        n = min(65535, n_tiles - first)
        _check(lib, lib.x0ne_attention_prefill_tcgen05(
            _ptr(q), _ptr(out), q.shape[0], cache, tile_seq.data_ptr() + 4 * first,
            tile_row0.data_ptr() + 4 * first, n, _ptr(seq_first_row), _ptr(seq_slot), _ptr(seq_pos0),
            q_heads, scale, window, _ptr(gemm_tc_status(q.device)), _stream()),
            "attention_prefill_tcgen05")


# ---------------------------------------------------------------------------------------------
# pass opener, per-head attention preparation without rotation, bias + activation (module `core`)
# ---------------------------------------------------------------------------------------------
def open_pass(resid: torch.Tensor, delta: Optional[torch.Tensor], table: Optional[torch.Tensor], tokens: Optional[torch.Tensor],
              scale: float, step: Optional[torch.Tensor], n_rows: int) -> None:
    """resid = ((resid + delta) + scale * table[tokens]) + step in float32; each term is optional."""
    lib = _lib("core")
    _need(resid, torch.float32, "residual")
    hidden = resid.shape[-1]
    if delta is not None:
        _need(delta, delta.dtype, "delta")
    if step is not None:
        _need(step, torch.float32, "step vector")
    if table is not None:
        _need(tokens, torch.int32, "tokens")
        _need(table, table.dtype, "embedding table")
    if resid.numel() < n_rows * hidden or (delta is not None and (delta.shape[-1] != hidden or delta.numel() < n_rows * hidden)) \
            or (step is not None and step.numel() != hidden) or (table is not None and (table.shape[-1] != hidden or tokens.numel() < n_rows)):
        raise KernelError("open_pass: widths or rows do not match")
    _check(lib, lib.x0ne_open_pass(_ptr(resid), _ptr(delta), dtype_tag(delta.dtype) if delta is not None else F32, _ptr(table),
                                   dtype_tag(table.dtype) if table is not None else F32, _ptr(tokens), float(scale), _ptr(step),
                                   n_rows, hidden, table.shape[0] if table is not None else 0, _stream()), "open_pass")


def head_norm_kv_write(src: torch.Tensor, k_col: int, v_col: int, q_norm: Optional[torch.Tensor], k_norm: Optional[torch.Tensor],
                       eps: float, temp_coef: float, temp_every: int, v_unit: bool, q_out: torch.Tensor, q_heads: int,
                       cache: PagedCacheArg, row_slot: torch.Tensor, row_pos: torch.Tensor, n_rows: int) -> None:
    """Per-head RMS norm of the queries (columns from 0) and keys (from k_col) of `src` with one weight of head_dim
    values each, the queries times 1 + temp_coef ln(floor((pos + 1) / temp_every) + 1) (temp_every 0: no such factor),
    the values (from v_col) brought to unit root mean square if `v_unit`; queries to q_out, keys and values to the pages."""
    lib = _lib("core")
    _need(src, src.dtype, "projection")
    _need(q_out, src.dtype, "queries")
    for t, what in ((q_norm, "query norm weight"), (k_norm, "key norm weight")):
        if t is not None:
            _need(t, torch.float32, what)
            if t.numel() != cache.head_dim:
                raise KernelError(f"head_norm_kv_write: the {what} does not have head_dim values")
    if src.numel() < n_rows * src.shape[-1] or q_out.shape[-1] != q_heads * cache.head_dim or q_out.numel() < n_rows * q_out.shape[-1]:
        raise KernelError("head_norm_kv_write: buffers smaller than the rows asked for")
    _check(lib, lib.x0ne_head_norm_kv_write(_ptr(src), dtype_tag(src.dtype), src.shape[-1], k_col, v_col, _ptr(q_norm), _ptr(k_norm),
                                            float(eps), float(temp_coef), int(temp_every or 0), 1 if v_unit else 0, _ptr(q_out), q_heads,
                                            cache, _ptr(row_slot), _ptr(row_pos), n_rows, _stream()), "head_norm_kv_write")


ACT_NONE, ACT_QUAD_EXP = 0, 1


def bias_act(x: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, n_rows: int, act: int = ACT_NONE, a: float = 0.0,
             b: float = 0.0) -> None:
    """out = act(x + bias) in float32.  ACT_QUAD_EXP: z > 0: a z^2 + z / 2; z <= 0: b (exp(z) - 1 - z) + z / 2."""
    lib = _lib("core")
    _need(x, x.dtype, "rows")
    _need(out, x.dtype, "activation output")
    width = x.shape[-1]
    if bias is not None:
        _need(bias, torch.float32, "bias")
        if bias.numel() != width:
            raise KernelError("bias_act: the bias does not have the rows' width")
    if out.shape[-1] != width or x.numel() < n_rows * width or out.numel() < n_rows * width:
        raise KernelError("bias_act: widths or rows do not match")
    _check(lib, lib.x0ne_bias_act(_ptr(x), _ptr(bias), _ptr(out), dtype_tag(x.dtype), n_rows, width, act, float(a), float(b), _stream()),
           "bias_act")


# ---------------------------------------------------------------------------------------------
# linear recurrence with a matrix state per head (csrc/wkv.cu, module `core`)
# ---------------------------------------------------------------------------------------------
def token_shift_mix(h: torch.Tensor, mu: torch.Tensor, mixes: torch.Tensor, state: torch.Tensor, last_off: int,
                    row_slot: torch.Tensor, row_pos: torch.Tensor, n_rows: int) -> None:
    """mixes[s, row] = h[row] + (h_before[row] - h[row]) * mu[s]: h_before is the row above where that is the same
    sequence's previous position, else the `width` values at `last_off` of the sequence's state row (zeros at a start)."""
    lib = _lib("core")
    _need(h, h.dtype, "mixer input")
    _need(mu, torch.float32, "mix coefficients")
    _need(mixes, h.dtype, "mixes")
    _need(state, torch.float32, "state")
    width = h.shape[-1]
    n_mix = mu.shape[0]
    if mu.shape[-1] != width or mixes.dim() != 3 or mixes.shape[0] != n_mix or mixes.shape[-1] != width or mixes.shape[1] < n_rows \
            or h.numel() < n_rows * width or state.dim() != 2 or state.shape[1] < last_off + width:
        raise KernelError("token_shift_mix: shapes do not match")
    _check(lib, lib.x0ne_token_shift_mix(_ptr(h), dtype_tag(h.dtype), _ptr(mu), n_mix, _ptr(mixes), mixes.stride(0), _ptr(state),
                                         state.stride(0), last_off, _ptr(row_slot), _ptr(row_pos), n_rows, width, _stream()),
           "token_shift_mix")


def wkv_scan(r: torch.Tensor, k: torch.Tensor, v: torch.Tensor, z: torch.Tensor, w0: torch.Tensor, u: torch.Tensor, h: torch.Tensor,
             o: torch.Tensor, state: torch.Tensor, seq_first_row: torch.Tensor, seq_slot: torch.Tensor, n_seqs: int, heads: int,
             n: int, one_token: bool = False) -> None:
    """Per sequence and head, token by token over the sequence's rows, from and into its state [heads, n, n]:
    w = exp(-exp(z + w0)); o[j] = sum_i r[i] (S[i][j] + u[i] k[i] v[j]); S[i][j] = w[i] S[i][j] + k[i] v[j].  The last
    row's h is left behind the matrices in the state row.  r, k, v, h in the activation type; z, o, state float32.
    `one_token`: every sequence brings one row (a decode step); the kernel made for that runs, with the same bits."""
    lib = _lib("core")
    for t, what in ((r, "r"), (k, "k"), (v, "v"), (h, "mixer input")):
        _need(t, r.dtype, what)
    for t, what in ((z, "decay exponents"), (w0, "decay offsets"), (u, "bonus"), (o, "scan output"), (state, "state")):
        _need(t, torch.float32, what)
    hn, width = heads * n, h.shape[-1]
    if any(t.shape[-1] != hn for t in (r, k, v, z, o)) or w0.numel() != hn or u.numel() != hn or state.dim() != 2 \
            or state.shape[1] < heads * n * n + width:
        raise KernelError("wkv_scan: shapes do not match")
    _check(lib, lib.x0ne_wkv_scan(_ptr(r), _ptr(k), _ptr(v), dtype_tag(r.dtype), _ptr(z), _ptr(w0), _ptr(u), _ptr(h), _ptr(o),
                                  _ptr(state), state.stride(0), _ptr(seq_first_row), _ptr(seq_slot), n_seqs, heads, n, width,
                                  1 if one_token else 0, _stream()), "wkv_scan")


def head_norm_gate(o: torch.Tensor, weight: torch.Tensor, gate: torch.Tensor, out: torch.Tensor, n_rows: int, heads: int, n: int,
                   eps: float) -> None:
    """out[row, head] = o / sqrt(mean(o^2) + eps) * weight * silu(gate), per head of n values; o float32."""
    lib = _lib("core")
    _need(o, torch.float32, "scan output")
    _need(weight, torch.float32, "head norm weight")
    _need(gate, gate.dtype, "gate")
    _need(out, gate.dtype, "gated output")
    hn = heads * n
    if o.shape[-1] != hn or gate.shape[-1] != hn or out.shape[-1] != hn or weight.numel() != hn or out.numel() < n_rows * hn:
        raise KernelError("head_norm_gate: shapes do not match")
    _check(lib, lib.x0ne_head_norm_gate(_ptr(o), _ptr(weight), _ptr(gate), _ptr(out), dtype_tag(out.dtype), n_rows, heads, n, float(eps),
                                        _stream()), "head_norm_gate")


def tanh_rows(x: torch.Tensor, out: torch.Tensor, n_rows: int) -> None:
    """out = tanh(x) for the first n_rows rows; x float32."""
    lib = _lib("core")
    _need(x, torch.float32, "rows")
    _need(out, out.dtype, "tanh output")
    if out.shape[-1] != x.shape[-1] or x.numel() < n_rows * x.shape[-1] or out.numel() < n_rows * x.shape[-1]:
        raise KernelError("tanh_rows: shapes do not match")
    _check(lib, lib.x0ne_tanh_rows(_ptr(x), _ptr(out), dtype_tag(out.dtype), n_rows * x.shape[-1], _stream()), "tanh_rows")


def rope_pairs_kv_write(src: torch.Tensor, k_col: int, v_col: int, freq: Optional[torch.Tensor], table: Optional[torch.Tensor], rot: int,
                        maps: int, dim: int, unit_eps: Optional[float], q_out: torch.Tensor, q_heads: int, q_padded: bool,
                        cache: PagedCacheArg, row_slot: torch.Tensor, row_pos: torch.Tensor, n_rows: int, write_kv: bool = True) -> None:
    """Queries (columns from 0), keys (from k_col) and values (from v_col) of the packed projection `src`: of every
    (head, map) of `dim` values the first `rot` turn as interleaved pairs by pos * freq[i] (`table`: float32
    [positions, rot], cosines then sines), then, with `unit_eps` not None, it is divided by its root mean square; queries
    to q_out ([rows, q_heads * maps, dim], or with `q_padded` [rows, q_heads * maps, maps * dim] with zeros beside the
    query's own map), keys (a kv head's maps side by side) and values to the pages."""
    lib = _lib("core")
    _need(src, src.dtype, "projection")
    _need(q_out, src.dtype, "queries")
    if freq is not None:
        _need(freq, torch.float32, "rotary frequencies")
    if table is not None:
        _need(table, torch.float32, "rotary table")
        if table.dim() != 2 or table.shape[1] != rot:
            raise KernelError("rope_pairs_kv_write: the table's rows do not hold rot values")
    if rot and (freq is None or freq.numel() < rot // 2):
        raise KernelError("rope_pairs_kv_write: fewer frequencies than pairs")
    q_width = q_heads * maps * (maps * dim if q_padded else dim)
    if src.numel() < n_rows * src.shape[-1] or q_out.shape[-1] != q_width or q_out.numel() < n_rows * q_width:
        raise KernelError("rope_pairs_kv_write: buffers smaller than the rows asked for")
    _check(lib, lib.x0ne_rope_pairs_kv_write(_ptr(src), dtype_tag(src.dtype), src.shape[-1], k_col, v_col, _ptr(freq), _ptr(table),
                                             0 if table is None else table.shape[0], rot, maps, dim,
                                             -1.0 if unit_eps is None else float(unit_eps), _ptr(q_out), q_heads, 1 if q_padded else 0,
                                             cache, _ptr(row_slot), _ptr(row_pos), n_rows, 1 if write_kv else 0, _stream()),
           "rope_pairs_kv_write")


def diff_heads(att: torch.Tensor, gate: Optional[torch.Tensor], gate_ld: int, out: torch.Tensor, n_rows: int, heads: int, vd: int,
               lam: float, eps: float, post: float) -> None:
    """out[row, head] = o / sqrt(mean(o^2) + eps) * post * sigmoid(gate[row, head]) with o = a1 - lam * a2, where att
    holds float32 [rows, heads, 2, vd] (the two maps' results of each head) and `gate`, of out's type, is a view whose
    row r starts gate_ld values after row r - 1 (None: no gate)."""
    lib = _lib("core")
    _need(att, torch.float32, "attention maps")
    _need(out, out.dtype, "combined heads")
    if att.shape[-1] != 2 * heads * vd or out.shape[-1] != heads * vd or att.numel() < n_rows * att.shape[-1] or out.numel() < n_rows * heads * vd:
        raise KernelError("diff_heads: shapes do not match")
    if gate is not None and (gate.dtype != out.dtype or not gate.is_cuda):
        raise KernelError("diff_heads: the gate is not of the output's type")
    _check(lib, lib.x0ne_diff_heads(_ptr(att), _ptr(gate), int(gate_ld), _ptr(out), dtype_tag(out.dtype), n_rows, heads, vd, float(lam),
                                    float(eps), float(post), _stream()), "diff_heads")


def causal_conv_silu(xz: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], state: torch.Tensor, conv_off: int, out: torch.Tensor,
                     row_slot: torch.Tensor, row_pos: torch.Tensor, n_rows: int, channels: int) -> None:
    """out[t, c] = silu(bias[c] + sum_k w[c, k] x[t - (K - 1 - k), c]) over the first `channels` columns of xz; inputs ahead of
    a row are the rows above it while they continue its sequence, then the K - 1 inputs its state row keeps at
    conv_off (float32 [K - 1, channels], oldest first).  The state is only read."""
    lib = _lib("core")
    _need(xz, xz.dtype, "convolution input")
    _need(out, xz.dtype, "convolution output")
    _need(w, torch.float32, "convolution taps")
    _need(state, torch.float32, "state")
    if bias is not None:
        _need(bias, torch.float32, "convolution bias")
    if w.dim() != 2 or w.shape[0] != channels or out.shape[-1] != channels or xz.shape[-1] < channels or state.dim() != 2 \
            or out.numel() < n_rows * channels or xz.numel() < n_rows * xz.shape[-1]:
        raise KernelError("causal_conv_silu: shapes do not match")
    _check(lib, lib.x0ne_causal_conv_silu(_ptr(xz), xz.shape[-1], dtype_tag(xz.dtype), _ptr(w), _ptr(bias), _ptr(state), state.stride(0),
                                          int(conv_off), _ptr(out), _ptr(row_slot), _ptr(row_pos), n_rows, channels, w.shape[1],
                                          _stream()), "causal_conv_silu")


def selective_scan(u: torch.Tensor, xz: torch.Tensor, z_col: int, dt_raw: torch.Tensor, dt_bias: Optional[torch.Tensor], A: torch.Tensor,
                   bc: torch.Tensor, b_col: int, c_col: int, D: Optional[torch.Tensor], out: torch.Tensor, state: torch.Tensor,
                   conv_off: int, taps: int, seq_first_row: torch.Tensor, seq_slot: torch.Tensor, n_seqs: int,
                   one_token: bool = False) -> None:
    """Per sequence and channel, token by token over the sequence's rows, from and into its state row (S [channels, N] at
    0, the convolution's last taps - 1 inputs at conv_off): dt = softplus(dt_raw + dt_bias); S = exp(dt A) S + dt u B;
    out = (S . C + D u) * silu(z).  u, xz (the convolution's input at column 0, z at z_col) and out in the activation type;
    dt_raw, A (negative), bc (B at b_col, C at c_col), D, state float32.  `one_token`: every sequence brings one row (a decode
    step); the same bits, from a form of the kernel without idle places."""
    lib = _lib("core")
    for t, what in ((u, "scan input"), (xz, "projection"), (out, "scan output")):
        _need(t, u.dtype, what)
    for t, what in ((dt_raw, "step sizes"), (A, "decay rates"), (bc, "B and C"), (state, "state")):
        _need(t, torch.float32, what)
    for t, what in ((dt_bias, "step size bias"), (D, "skip weights")):
        if t is not None:
            _need(t, torch.float32, what)
    channels, N = A.shape
    if u.shape[-1] != channels or out.shape[-1] != channels or dt_raw.shape[-1] != channels or state.dim() != 2 \
            or (dt_bias is not None and dt_bias.numel() != channels) or (D is not None and D.numel() != channels):
        raise KernelError("selective_scan: shapes do not match")
    arg = SsmArg(_ptr(u), _ptr(xz), xz.shape[-1], int(z_col), _ptr(dt_raw), _ptr(dt_bias), _ptr(A), _ptr(bc), bc.shape[-1], int(b_col),
                 int(c_col), _ptr(D), _ptr(out), _ptr(state), state.stride(0), int(conv_off), _ptr(seq_first_row), _ptr(seq_slot),
                 int(channels), int(N), int(taps))
    _check(lib, lib.x0ne_selective_scan(arg, dtype_tag(u.dtype), n_seqs, 1 if one_token else 0, _stream()), "selective_scan")
