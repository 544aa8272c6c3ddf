"""Thin tensor-level wrappers over the C ABI (one function per entry point).

They validate dtype / device / contiguity, allocate outputs with torch and launch on the
current stream.  Nothing here computes on the CPU.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence, Tuple

import torch

from . import _lib
from ._lib import check, ptr, require_cuda, status_word, stream_ptr

NEG_INF = float("-inf")


def _i32(t: Optional[torch.Tensor], name: str) -> Optional[torch.Tensor]:
    if t is None:
        return None
    if t.dtype != torch.int32 or not t.is_contiguous():
        raise _lib.B200DSAError(f"{name} must be a contiguous int32 tensor")
    return t


def topk_select(scores: torch.Tensor, k: int, *, col_begin: Optional[torch.Tensor] = None,
                col_end: Optional[torch.Tensor] = None, keep_pos_inf: bool = False,
                pos_map: Optional[torch.Tensor] = None, page_table: Optional[torch.Tensor] = None,
                page_size: int = 0, row_pos_offset: Optional[torch.Tensor] = None,
                sorted: bool = True, return_values: bool = False, out: Optional[torch.Tensor] = None,
                out_values: Optional[torch.Tensor] = None, seg_cols: int = 0, seg_stride: int = 0,
                n_cols: Optional[int] = None, row_stride: Optional[int] = None,
                n_rows: Optional[int] = None, pos_map_stride: Optional[int] = None,
                seg_offsets: Optional[Sequence[int]] = None):
    """Row-wise top-k positions (int32, -1 padded; descending score when sorted); see
    b200dsa_topk_select.  seg_offsets: element offsets of the segments from scores / pos_map
    (segments in separate, possibly peer-GPU, buffers)."""
    require_cuda(scores, col_begin, col_end, pos_map, page_table, row_pos_offset)
    if scores.dtype != torch.float32 or scores.dim() != 2 or scores.stride(1) != 1:
        raise _lib.B200DSAError("scores must be a 2-D fp32 tensor with unit column stride")
    n_rows = scores.shape[0] if n_rows is None else n_rows
    n_cols = scores.shape[1] if n_cols is None else n_cols
    row_stride = scores.stride(0) if row_stride is None else row_stride
    if out is None:
        out = torch.empty(n_rows, k, dtype=torch.int32, device=scores.device)
    elif out.dtype != torch.int32 or out.stride(1) != 1 or out.shape[0] < n_rows or out.shape[1] < k:
        raise _lib.B200DSAError("out must be int32 [>=n_rows, >=k] with unit column stride")
    vals = out_values
    if vals is None and return_values:
        vals = torch.empty(n_rows, out.stride(0), dtype=torch.float32, device=scores.device)
    if vals is not None and (vals.dtype != torch.float32 or vals.stride(0) != out.stride(0)):
        raise _lib.B200DSAError("out_values must be fp32 with the row stride of out")
    seg_arr = (ctypes.c_int64 * len(seg_offsets))(*seg_offsets) if seg_offsets is not None else None
    lib = _lib.load()
    rc = lib.b200dsa_topk_select(
        ptr(scores), row_stride, n_rows, n_cols,
        ptr(_i32(col_begin, "col_begin")), ptr(_i32(col_end, "col_end")), k, int(keep_pos_inf), int(sorted),
        ptr(_i32(pos_map, "pos_map")),
        (pos_map_stride if pos_map_stride is not None else pos_map.stride(0)) if pos_map is not None else 0,
        ptr(_i32(page_table, "page_table")), page_table.stride(0) if page_table is not None else 0, page_size,
        ptr(_i32(row_pos_offset, "row_pos_offset")), seg_cols, seg_stride, seg_arr,
        ptr(out), ptr(vals), out.stride(0), stream_ptr())
    check(rc, "b200dsa_topk_select")
    if return_values or out_values is not None:
        return out[:n_rows, :k], vals[:n_rows, :k]
    return out[:n_rows, :k]


CAND_CAP = 8192  # candidate list entries per row of the split top-k scratch


def _check_topk_outputs(out: torch.Tensor, out_values: Optional[torch.Tensor], n_rows: int, k: int) -> None:
    """The kernels write row r of both outputs at r * out.stride(0): shapes, dtypes and strides must agree."""
    if out.dtype != torch.int32 or out.dim() != 2 or out.stride(1) != 1 or out.shape[0] < n_rows or out.shape[1] < k:
        raise _lib.B200DSAError("out must be int32 [>=n_rows, >=k] with unit column stride")
    if out_values is not None and (out_values.dtype != torch.float32 or out_values.dim() != 2 or
                                   out_values.stride(1) != 1 or out_values.stride(0) != out.stride(0) or
                                   out_values.shape[0] < n_rows or out_values.shape[1] < k):
        raise _lib.B200DSAError("out_values must be fp32 [>=n_rows, >=k] with the row stride of out")


def topk_scratch(n_rows: int, device) -> Tuple[torch.Tensor, torch.Tensor]:
    """Scratch for topk_select_split: (candidates uint64-as-int64 [n_rows, 8192], zeroed int32 [2*n_rows]:
    per-row counters then per-row bin floors).  Only the counters have to start at zero."""
    return (torch.empty(n_rows, CAND_CAP, dtype=torch.int64, device=device),
            torch.zeros(2 * n_rows, dtype=torch.int32, device=device))


FUSED_CAND_CAP = 16384  # candidate list entries per row that the indexer's epilogue may collect


def fused_scratch(n_rows: int, device) -> Tuple[torch.Tensor, torch.Tensor]:
    """Scratch for indexer_paged_fp8_topk: (candidates uint64-as-int64 [n_rows, 16384], zeroed int32
    [2*n_rows]: per-row counters then per-row floors).  Both halves of the int32 part must be zero before
    the first call; every call leaves them zero.  Not interchangeable with topk_scratch()."""
    return (torch.empty(n_rows, FUSED_CAND_CAP, dtype=torch.int64, device=device),
            torch.zeros(2 * n_rows, dtype=torch.int32, device=device))


_scratch_cache = {}


def topk_scratch_cached(n_rows: int, device) -> Tuple[torch.Tensor, torch.Tensor]:
    """One scratch pair per (device, row count), allocated on first use and kept: callers that run
    every step (routers, the serving hook) must not allocate and zero-fill per call.  Calls that
    share it must not overlap on the GPU (same stream, or ordered by events)."""
    dev = torch.device(device)
    key = (dev.type, dev.index if dev.index is not None else torch.cuda.current_device(), n_rows)
    if key not in _scratch_cache:
        _scratch_cache[key] = topk_scratch(n_rows, dev)
    return _scratch_cache[key]


def fused_scratch_cached(n_rows: int, device) -> Tuple[torch.Tensor, torch.Tensor]:
    """fused_scratch() kept per (device, row count); the same sharing rule as topk_scratch_cached."""
    dev = torch.device(device)
    key = ("fused", dev.type, dev.index if dev.index is not None else torch.cuda.current_device(), n_rows)
    if key not in _scratch_cache:
        _scratch_cache[key] = fused_scratch(n_rows, dev)
    return _scratch_cache[key]


def topk_select_split(scores: torch.Tensor, k: int, scratch: Tuple[torch.Tensor, torch.Tensor], *,
                      col_begin: Optional[torch.Tensor] = None, col_end: Optional[torch.Tensor] = None,
                      keep_pos_inf: bool = False, row_pos_offset: Optional[torch.Tensor] = None,
                      sorted: bool = True, splits: int = 0, out: Optional[torch.Tensor] = None,
                      out_values: Optional[torch.Tensor] = None):
    """Top-k for few long rows, several CTAs per row; see b200dsa_topk_select_split.  `scratch`
    comes from topk_scratch() and may be reused by later calls on the same stream."""
    require_cuda(scores, col_begin, col_end, row_pos_offset, *scratch)
    if scores.dtype != torch.float32 or scores.dim() != 2 or scores.stride(1) != 1:
        raise _lib.B200DSAError("scores must be a 2-D fp32 tensor with unit column stride")
    n_rows, n_cols = scores.shape
    cand, count = scratch
    if cand.numel() < n_rows * CAND_CAP or count.numel() < 2 * n_rows:
        raise _lib.B200DSAError("scratch is too small for this many rows")
    if splits <= 0:
        splits = max(1, min(16, (2 * 148) // max(1, n_rows)))
    if out is None:
        out = torch.empty(n_rows, k, dtype=torch.int32, device=scores.device)
    _check_topk_outputs(out, out_values, n_rows, k)
    rc = _lib.load().b200dsa_topk_select_split(
        ptr(scores), scores.stride(0), n_rows, n_cols, ptr(_i32(col_begin, "col_begin")),
        ptr(_i32(col_end, "col_end")), k, int(keep_pos_inf), int(sorted), ptr(_i32(row_pos_offset, "row_pos_offset")),
        splits, ptr(cand), ptr(count), ptr(out), ptr(out_values), out.stride(0), stream_ptr())
    check(rc, "b200dsa_topk_select_split")
    if out_values is not None:
        return out[:n_rows, :k], out_values[:n_rows, :k]
    return out[:n_rows, :k]


STATIC_TOPK_MAX_ROWS = 64


def topk_select_split_static(scores: torch.Tensor, k: int, *, col_begin: Optional[torch.Tensor] = None,
                             col_end: Optional[torch.Tensor] = None, keep_pos_inf: bool = False,
                             row_pos_offset: Optional[torch.Tensor] = None, sorted: bool = True, splits: int = 0,
                             out: torch.Tensor = None, out_values: Optional[torch.Tensor] = None):
    """topk_select_split on the library's built-in scratch (at most 64 rows): for callers that
    have no device memory to lend.  `out` (int32 [n_rows, >=k]) must be supplied, so that this
    wrapper, like the entry point under it, allocates nothing.  One call at a time per device."""
    require_cuda(scores, col_begin, col_end, row_pos_offset, out, out_values)
    if scores.dtype != torch.float32 or scores.dim() != 2 or scores.stride(1) != 1:
        raise _lib.B200DSAError("scores must be a 2-D fp32 tensor with unit column stride")
    if out is None:
        raise _lib.B200DSAError("out must be a preallocated int32 [n_rows, >=k] tensor")
    n_rows, n_cols = scores.shape
    _check_topk_outputs(out, out_values, n_rows, k)
    if splits <= 0:
        splits = max(1, min(16, (2 * 148) // max(1, n_rows)))
    rc = _lib.load().b200dsa_topk_select_split_static(
        ptr(scores), scores.stride(0), n_rows, n_cols, ptr(_i32(col_begin, "col_begin")),
        ptr(_i32(col_end, "col_end")), k, int(keep_pos_inf), int(sorted), ptr(_i32(row_pos_offset, "row_pos_offset")),
        splits, ptr(out), ptr(out_values), out.stride(0), stream_ptr())
    check(rc, "b200dsa_topk_select_split_static")
    if out_values is not None:
        return out[:n_rows, :k], out_values[:n_rows, :k]
    return out[:n_rows, :k]


def indexer_paged_fp8_logits(q_fp8: torch.Tensor, weights: torch.Tensor, cache: torch.Tensor, page_size: int,
                             context_lens: torch.Tensor, block_table: torch.Tensor, *, next_n: int = 1,
                             max_cols: Optional[int] = None, out_scale: float = 1.0,
                             out: Optional[torch.Tensor] = None, fill: bool = True,
                             row_table: Optional[torch.Tensor] = None, head_mask: Optional[torch.Tensor] = None,
                             out_gated: Optional[torch.Tensor] = None):
    """Decode logits [n_rows, max_cols] fp32 over the paged FP8 cache; see
    b200dsa_indexer_paged_fp8_logits.  fill=True pre-fills a fresh output with -inf so that
    columns beyond each context are -inf as in the reference; pass out= to reuse a buffer.
    With head_mask (int64 [n_rows], bit h = head h) the same pass also produces the sum over the
    masked heads only, and the call returns (logits, gated logits)."""
    require_cuda(q_fp8, weights, cache, context_lens, block_table, head_mask, out_gated)
    if q_fp8.dtype != torch.float8_e4m3fn or not q_fp8.is_contiguous() or q_fp8.shape[-2:] != (64, 128):
        raise _lib.B200DSAError("q_fp8 must be contiguous float8_e4m3fn [..., 64, 128]")
    n_rows = q_fp8.numel() // (64 * 128)
    if weights.dtype != torch.float32 or not weights.is_contiguous() or weights.numel() != n_rows * 64:
        raise _lib.B200DSAError("weights must be contiguous fp32 [n_rows, 64]")
    if cache.dtype != torch.uint8 or not cache.is_contiguous():
        raise _lib.B200DSAError("cache must be a contiguous uint8 tensor")
    page_bytes = page_size * 132
    if cache.numel() % page_bytes:
        raise _lib.B200DSAError("cache size is not a multiple of page_size*(128+4)")
    num_pages = cache.numel() // page_bytes
    _i32(context_lens, "context_lens"); _i32(block_table, "block_table")
    if context_lens.numel() != n_rows:
        raise _lib.B200DSAError("context_lens must have one entry per row")
    if max_cols is None:
        max_cols = block_table.shape[-1] * page_size
    if out is None:
        out = (torch.full if fill else torch.empty)(
            (n_rows, max_cols), *((NEG_INF,) if fill else ()), dtype=torch.float32, device=q_fp8.device)
    out_gated = _gated_output(head_mask, out_gated, out, n_rows, fill)
    lib = _lib.load()
    rc = lib.b200dsa_indexer_paged_fp8_logits(
        ptr(q_fp8), ptr(weights), ptr(cache), num_pages, page_size, ptr(context_lens),
        ptr(block_table), block_table.stride(0), ptr(_i32(row_table, "row_table")), n_rows, next_n, max_cols,
        out_scale,
        ptr(out), out.stride(0), ptr(head_mask), ptr(out_gated), ptr(status_word(q_fp8.device)), stream_ptr())
    check(rc, "b200dsa_indexer_paged_fp8_logits")
    return out if head_mask is None else (out, out_gated)


def indexer_paged_blocklist_fp8_logits(q_fp8: torch.Tensor, weights: torch.Tensor, cache: torch.Tensor, page_size: int,
                                       context_lens: torch.Tensor, block_table: torch.Tensor,
                                       block_list: torch.Tensor, row_cols: torch.Tensor, *, next_n: int = 1,
                                       out_scale: float = 1.0, row_table: Optional[torch.Tensor] = None,
                                       out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Token logits [n_rows, 128*list_len] inside per-row lists of 128-key blocks of the paged FP8 cache
    (-inf for unlisted / masked columns); see b200dsa_indexer_paged_blocklist_fp8_logits."""
    require_cuda(q_fp8, weights, cache, context_lens, block_table, block_list, row_cols, row_table, out)
    if q_fp8.dtype != torch.float8_e4m3fn or not q_fp8.is_contiguous() or q_fp8.shape[-2:] != (64, 128):
        raise _lib.B200DSAError("q_fp8 must be contiguous float8_e4m3fn [..., 64, 128]")
    n_rows = q_fp8.numel() // (64 * 128)
    if weights.dtype != torch.float32 or not weights.is_contiguous() or weights.numel() != n_rows * 64:
        raise _lib.B200DSAError("weights must be contiguous fp32 [n_rows, 64]")
    if cache.dtype != torch.uint8 or not cache.is_contiguous() or cache.numel() % (page_size * 132):
        raise _lib.B200DSAError("cache must be contiguous uint8 with page_size*(128+4) bytes per page")
    num_pages = cache.numel() // (page_size * 132)
    for t_, nm in ((context_lens, "context_lens"), (block_table, "block_table"), (block_list, "block_list"),
                   (row_cols, "row_cols")):
        _i32(t_, nm)
    if block_list.dim() != 2 or block_list.shape[0] != n_rows or context_lens.numel() != n_rows or \
            row_cols.numel() != n_rows:
        raise _lib.B200DSAError("block_list must be [n_rows, list_len]; context_lens and row_cols one entry per row")
    max_cols = block_list.shape[1] * 128
    if out is None:
        out = torch.full((n_rows, max_cols), NEG_INF, dtype=torch.float32, device=q_fp8.device)
    elif out.dtype != torch.float32 or out.stride(1) != 1 or out.shape[0] < n_rows or out.shape[1] < max_cols:
        raise _lib.B200DSAError("out must be fp32 [>=n_rows, >=128*list_len] with unit column stride")
    rc = _lib.load().b200dsa_indexer_paged_blocklist_fp8_logits(
        ptr(q_fp8), ptr(weights), ptr(cache), num_pages, page_size, ptr(context_lens), ptr(block_table),
        block_table.stride(0), ptr(_i32(row_table, "row_table")), n_rows, next_n, ptr(block_list),
        block_list.stride(0), ptr(row_cols), max_cols, out_scale, ptr(out), out.stride(0),
        ptr(status_word(q_fp8.device)), stream_ptr())
    check(rc, "b200dsa_indexer_paged_blocklist_fp8_logits")
    return out


def indexer_paged_fp8_topk(q_fp8: torch.Tensor, weights: torch.Tensor, cache: torch.Tensor, page_size: int,
                           context_lens: torch.Tensor, block_table: torch.Tensor, k: int,
                           scratch: Tuple[torch.Tensor, torch.Tensor], *, next_n: int = 1,
                           max_cols: Optional[int] = None, out_scale: float = 1.0,
                           logits: Optional[torch.Tensor] = None, keep_logits: bool = True,
                           row_table: Optional[torch.Tensor] = None, row_pos_offset: Optional[torch.Tensor] = None,
                           sorted: bool = False, out: Optional[torch.Tensor] = None,
                           out_values: Optional[torch.Tensor] = None, push=None):
    """Indexer scores and their top-k positions in two launches, the candidates collected by the
    indexer's own epilogue; see b200dsa_indexer_paged_fp8_topk.  `scratch` comes from fused_scratch().
    keep_logits=True (default) also writes the logits (into `logits`, allocated when not given) so
    that a row whose candidate list is not provably complete is selected exactly from them;
    keep_logits=False writes no logits at all (status word 3 on such a row).
    push=(link, off_recv): the selection also stores its rows into every peer's receive area and
    raises this rank's flag (b200dsa_indexer_paged_fp8_topk_push; link from PeerLseCombine.link())."""
    require_cuda(q_fp8, weights, cache, context_lens, block_table, row_table, row_pos_offset, logits, out, out_values)
    if q_fp8.dtype != torch.float8_e4m3fn or not q_fp8.is_contiguous() or q_fp8.shape[-2:] != (64, 128):
        raise _lib.B200DSAError("q_fp8 must be contiguous float8_e4m3fn [..., 64, 128]")
    n_rows = q_fp8.numel() // (64 * 128)
    if weights.dtype != torch.float32 or not weights.is_contiguous() or weights.numel() != n_rows * 64:
        raise _lib.B200DSAError("weights must be contiguous fp32 [n_rows, 64]")
    if cache.dtype != torch.uint8 or not cache.is_contiguous() or cache.numel() % (page_size * 132):
        raise _lib.B200DSAError("cache must be contiguous uint8 with page_size*(128+4) bytes per page")
    num_pages = cache.numel() // (page_size * 132)
    _i32(context_lens, "context_lens"); _i32(block_table, "block_table")
    if context_lens.numel() != n_rows:
        raise _lib.B200DSAError("context_lens must have one entry per row")
    if not 1 <= k <= 2048:
        raise _lib.B200DSAError("the fused selection supports 1 <= k <= 2048")
    if max_cols is None:
        max_cols = block_table.shape[-1] * page_size
    cand, count = scratch
    if cand.numel() < n_rows * FUSED_CAND_CAP or count.numel() < 2 * n_rows:
        raise _lib.B200DSAError("scratch is too small for this many rows (use fused_scratch())")
    if keep_logits and logits is None:
        logits = torch.empty(n_rows, max_cols, dtype=torch.float32, device=q_fp8.device)
    if not keep_logits:
        logits = None
    if logits is not None and (logits.dtype != torch.float32 or logits.stride(1) != 1 or logits.shape[0] < n_rows or
                               logits.shape[1] < max_cols):
        raise _lib.B200DSAError("logits must be fp32 [>=n_rows, >=max_cols] with unit column stride")
    if out is None:
        out = torch.empty(n_rows, k, dtype=torch.int32, device=q_fp8.device)
    _check_topk_outputs(out, out_values, n_rows, k)
    args = (ptr(q_fp8), ptr(weights), ptr(cache), num_pages, page_size, ptr(context_lens), ptr(block_table),
            block_table.stride(0), ptr(_i32(row_table, "row_table")), n_rows, next_n, max_cols, out_scale, ptr(logits),
            logits.stride(0) if logits is not None else 0, k, int(sorted), ptr(_i32(row_pos_offset, "row_pos_offset")),
            ptr(cand), ptr(count), ptr(out), ptr(out_values), out.stride(0))
    if push is None:
        rc = _lib.load().b200dsa_indexer_paged_fp8_topk(*args, ptr(status_word(q_fp8.device)), stream_ptr())
    else:
        link, off_recv = push
        rc = _lib.load().b200dsa_indexer_paged_fp8_topk_push(*args, ctypes.byref(link), off_recv,
                                                             ptr(status_word(q_fp8.device)), stream_ptr())
    check(rc, "b200dsa_indexer_paged_fp8_topk")
    if out_values is not None:
        return out[:n_rows, :k], out_values[:n_rows, :k]
    return out[:n_rows, :k]


def _gated_output(head_mask, out_gated, out, n_rows, fill=True):
    if head_mask is None:
        if out_gated is not None:
            raise _lib.B200DSAError("out_gated needs head_mask")
        return None
    if head_mask.dtype != torch.int64 or not head_mask.is_contiguous() or head_mask.numel() != n_rows:
        raise _lib.B200DSAError("head_mask must be contiguous int64 [n_rows]")
    if out_gated is None:
        out_gated = torch.full_like(out, NEG_INF) if fill else torch.empty_like(out)
    if out_gated.dtype != torch.float32 or out_gated.shape != out.shape or out_gated.stride() != out.stride():
        raise _lib.B200DSAError("out_gated must have the shape and strides of the logits")
    return out_gated


def head_mask_from_indices(head_idx: torch.Tensor) -> torch.Tensor:
    """int64 [n_rows] bit masks (bit h = head h) from kept-head indices [n_rows, n_keep]."""
    keep = torch.zeros(head_idx.shape[0], 64, dtype=torch.bool, device=head_idx.device)
    keep.scatter_(1, head_idx.long(), True)
    bits = torch.bitwise_left_shift(keep.long(), torch.arange(64, device=head_idx.device))
    return bits.sum(dim=1)                      # distinct bits: the wrap-around of bit 63 is the bit pattern


def indexer_blocklist_bf16_logits(q: torch.Tensor, weights: torch.Tensor, keys: torch.Tensor,
                                  block_list: torch.Tensor, row_cols: torch.Tensor, *,
                                  pos_lo: Optional[torch.Tensor] = None, pos_hi: Optional[torch.Tensor] = None,
                                  out_scale: float = 1.0, out: Optional[torch.Tensor] = None,
                                  head_mask: Optional[torch.Tensor] = None,
                                  out_gated: Optional[torch.Tensor] = None, max_cols: Optional[int] = None):
    """Token logits [n_rows, 128*list_len] inside per-row lists of 128-key blocks; see
    b200dsa_indexer_blocklist_bf16_logits.  head_mask: as for indexer_paged_fp8_logits.
    block_list=None: row r covers consecutive blocks starting at the one that holds pos_lo[r]
    (pos_lo / pos_hi and max_cols, a multiple of 128, are then required)."""
    require_cuda(q, weights, keys, block_list, row_cols, pos_lo, pos_hi, head_mask, out_gated)
    if q.dtype != torch.bfloat16 or not q.is_contiguous() or q.shape[-2:] != (64, 128):
        raise _lib.B200DSAError("q must be contiguous bf16 [n_rows, 64, 128]")
    if keys.dtype != torch.bfloat16 or not keys.is_contiguous() or keys.shape[-1] != 128:
        raise _lib.B200DSAError("keys must be contiguous bf16 [n_keys, 128]")
    n_rows = q.shape[0]
    if weights.dtype != torch.float32 or not weights.is_contiguous() or weights.numel() != n_rows * 64:
        raise _lib.B200DSAError("weights must be contiguous fp32 [n_rows, 64]")
    _i32(block_list, "block_list"); _i32(row_cols, "row_cols")
    if block_list is None:
        if pos_lo is None or pos_hi is None or (max_cols is None and out is None):
            raise _lib.B200DSAError("without a block list pos_lo, pos_hi and max_cols are required")
        max_cols = out.shape[1] if max_cols is None else max_cols
    else:
        max_cols = block_list.shape[1] * 128
    if out is None:
        out = torch.full((n_rows, max_cols), NEG_INF, dtype=torch.float32, device=q.device)
    out_gated = _gated_output(head_mask, out_gated, out, n_rows)
    lib = _lib.load()
    rc = lib.b200dsa_indexer_blocklist_bf16_logits(
        ptr(q), ptr(weights), ptr(keys), keys.shape[0], ptr(block_list),
        block_list.stride(0) if block_list is not None else 0,
        ptr(row_cols), ptr(_i32(pos_lo, "pos_lo")), ptr(_i32(pos_hi, "pos_hi")), n_rows, max_cols, out_scale,
        ptr(out), out.stride(0), ptr(head_mask), ptr(out_gated), ptr(status_word(q.device)), stream_ptr())
    check(rc, "b200dsa_indexer_blocklist_bf16_logits")
    return out if head_mask is None else (out, out_gated)


def indexer_flat_bf16_logits(q: torch.Tensor, weights: torch.Tensor, keys: torch.Tensor, pos_lo: torch.Tensor,
                             pos_hi: torch.Tensor, row_cols: torch.Tensor, max_cols: int, *, out_scale: float = 1.0,
                             out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Prefill token logits [n_rows, max_cols] over flat bf16 keys, four queries per key tile; see
    b200dsa_indexer_flat_bf16_logits (column c of row r = position 128*(pos_lo[r]//128) + c)."""
    require_cuda(q, weights, keys, pos_lo, pos_hi, row_cols, out)
    if q.dtype != torch.bfloat16 or not q.is_contiguous() or q.shape[-2:] != (64, 128):
        raise _lib.B200DSAError("q must be contiguous bf16 [n_rows, 64, 128]")
    if keys.dtype != torch.bfloat16 or not keys.is_contiguous() or keys.shape[-1] != 128:
        raise _lib.B200DSAError("keys must be contiguous bf16 [n_keys, 128]")
    n_rows = q.shape[0]
    if weights.dtype != torch.float32 or not weights.is_contiguous() or weights.numel() != n_rows * 64:
        raise _lib.B200DSAError("weights must be contiguous fp32 [n_rows, 64]")
    for t_, nm in ((pos_lo, "pos_lo"), (pos_hi, "pos_hi"), (row_cols, "row_cols")):
        if _i32(t_, nm).numel() != n_rows:
            raise _lib.B200DSAError(f"{nm} must have one entry per row")
    if out is None:
        out = torch.full((n_rows, max_cols), NEG_INF, dtype=torch.float32, device=q.device)
    elif out.dtype != torch.float32 or out.stride(1) != 1 or out.shape[0] < n_rows or out.shape[1] < max_cols:
        raise _lib.B200DSAError("out must be fp32 [>=n_rows, >=max_cols] with unit column stride")
    rc = _lib.load().b200dsa_indexer_flat_bf16_logits(
        ptr(q), ptr(weights), ptr(keys), keys.shape[0], ptr(pos_lo), ptr(pos_hi), ptr(row_cols), n_rows, max_cols,
        out_scale, ptr(out), out.stride(0), ptr(status_word(q.device)), stream_ptr())
    check(rc, "b200dsa_indexer_flat_bf16_logits")
    return out


def causal_row_intervals(cu_seqlens: torch.Tensor, n_rows: int, q_pos: Optional[torch.Tensor] = None):
    """(lo, hi, col0, row_cols) int32 [n_rows] of packed causal queries in one launch; see
    b200dsa_causal_row_intervals."""
    require_cuda(cu_seqlens, q_pos)
    cu = cu_seqlens.to(torch.int32).contiguous()
    qp = None if q_pos is None else q_pos.to(torch.int32).contiguous()
    if qp is not None and qp.numel() != n_rows:
        raise _lib.B200DSAError("q_pos must have one entry per row")
    out = torch.empty(4, max(n_rows, 1), dtype=torch.int32, device=cu.device)
    rc = _lib.load().b200dsa_causal_row_intervals(ptr(cu), cu.numel(), ptr(qp), n_rows, ptr(out[0]), ptr(out[1]),
                                                   ptr(out[2]), ptr(out[3]), stream_ptr())
    check(rc, "b200dsa_causal_row_intervals")
    return out[0, :n_rows], out[1, :n_rows], out[2, :n_rows], out[3, :n_rows]


def indexer_flat_bf16_logits_routed(q8: torch.Tensor, weights8: torch.Tensor, keys: torch.Tensor, pos_lo: torch.Tensor,
                                    pos_hi: torch.Tensor, row_cols: torch.Tensor, max_cols: int, *,
                                    out_scale: float = 1.0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Routed prefill logits [n_rows, max_cols]: q8 [n_rows, 8, 128] are the eight heads kept for each query,
    32 queries per key tile; see b200dsa_indexer_flat_bf16_logits_routed (columns as in the all-head form)."""
    require_cuda(q8, weights8, keys, pos_lo, pos_hi, row_cols, out)
    if q8.dtype != torch.bfloat16 or not q8.is_contiguous() or q8.shape[-2:] != (8, 128):
        raise _lib.B200DSAError("q8 must be contiguous bf16 [n_rows, 8, 128]")
    if keys.dtype != torch.bfloat16 or not keys.is_contiguous() or keys.shape[-1] != 128:
        raise _lib.B200DSAError("keys must be contiguous bf16 [n_keys, 128]")
    n_rows = q8.shape[0]
    if weights8.dtype != torch.float32 or not weights8.is_contiguous() or weights8.numel() != n_rows * 8:
        raise _lib.B200DSAError("weights8 must be contiguous fp32 [n_rows, 8]")
    for t_, nm in ((pos_lo, "pos_lo"), (pos_hi, "pos_hi"), (row_cols, "row_cols")):
        if _i32(t_, nm).numel() != n_rows:
            raise _lib.B200DSAError(f"{nm} must have one entry per row")
    if out is None:
        out = torch.full((n_rows, max_cols), NEG_INF, dtype=torch.float32, device=q8.device)
    elif out.dtype != torch.float32 or out.stride(1) != 1 or out.shape[0] < n_rows or out.shape[1] < max_cols:
        raise _lib.B200DSAError("out must be fp32 [>=n_rows, >=max_cols] with unit column stride")
    rc = _lib.load().b200dsa_indexer_flat_bf16_logits_routed(
        ptr(q8), ptr(weights8), ptr(keys), keys.shape[0], ptr(pos_lo), ptr(pos_hi), ptr(row_cols), n_rows, max_cols,
        out_scale, ptr(out), out.stride(0), ptr(status_word(q8.device)), stream_ptr())
    check(rc, "b200dsa_indexer_flat_bf16_logits_routed")
    return out


def indexer_gather_bf16_logits(q: torch.Tensor, weights: torch.Tensor, keys: torch.Tensor, cand: torch.Tensor, *,
                               row_cols: Optional[torch.Tensor] = None, pos_lo: Optional[torch.Tensor] = None,
                               pos_hi: Optional[torch.Tensor] = None, out_scale: float = 1.0,
                               out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """All-head logits [n_rows, n_cand] of every query on its own candidate positions cand int32
    [n_rows, n_cand] (-1 = none -> -inf); see b200dsa_indexer_gather_bf16_logits."""
    require_cuda(q, weights, keys, cand, row_cols, pos_lo, pos_hi, out)
    if q.dtype != torch.bfloat16 or not q.is_contiguous() or q.shape[-2:] != (64, 128):
        raise _lib.B200DSAError("q must be contiguous bf16 [n_rows, 64, 128]")
    if keys.dtype != torch.bfloat16 or not keys.is_contiguous() or keys.shape[-1] != 128:
        raise _lib.B200DSAError("keys must be contiguous bf16 [n_keys, 128]")
    n_rows = q.shape[0]
    if weights.dtype != torch.float32 or not weights.is_contiguous() or weights.numel() != n_rows * 64:
        raise _lib.B200DSAError("weights must be contiguous fp32 [n_rows, 64]")
    if _i32(cand, "cand").dim() != 2 or cand.shape[0] != n_rows or cand.stride(1) != 1:
        raise _lib.B200DSAError("cand must be int32 [n_rows, n_cand] with unit column stride")
    n_cand = cand.shape[1]
    if row_cols is None:
        row_cols = torch.full((n_rows,), n_cand, dtype=torch.int32, device=q.device)
    for t_, nm in ((row_cols, "row_cols"), (pos_lo, "pos_lo"), (pos_hi, "pos_hi")):
        if t_ is not None and _i32(t_, nm).numel() != n_rows:
            raise _lib.B200DSAError(f"{nm} must have one entry per row")
    if out is None:
        out = torch.full((n_rows, n_cand), NEG_INF, dtype=torch.float32, device=q.device)
    elif out.dtype != torch.float32 or out.stride(1) != 1 or out.shape[0] < n_rows or out.shape[1] < n_cand:
        raise _lib.B200DSAError("out must be fp32 [>=n_rows, >=n_cand] with unit column stride")
    rc = _lib.load().b200dsa_indexer_gather_bf16_logits(
        ptr(q), ptr(weights), ptr(keys), keys.shape[0], ptr(cand), cand.stride(0), ptr(row_cols), ptr(pos_lo),
        ptr(pos_hi), n_rows, n_cand, out_scale, ptr(out), out.stride(0), ptr(status_word(q.device)), stream_ptr())
    check(rc, "b200dsa_indexer_gather_bf16_logits")
    return out


def sparse_mla_decode(q: torch.Tensor, kv: torch.Tensor, indices: torch.Tensor, sm_scale: float, *,
                      kv_row_base: Optional[torch.Tensor] = None, q_pos: Optional[torch.Tensor] = None,
                      pos_lo: int = 0, pos_hi: int = 2 ** 31 - 1, n_idx_item: Optional[torch.Tensor] = None,
                      ctx: Optional[torch.Tensor] = None, lse: Optional[torch.Tensor] = None,
                      q_pos_bias: int = 0, signal=None, pair: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """Latent-space sparse attention: (ctx [n, H, 512], lse [n, H] fp32); see
    b200dsa_sparse_mla_decode.  ctx is fp32 unless a bf16 buffer is passed in; q_pos_bias is added to
    q_pos (-1: q_pos holds context lengths).  signal=(link, ticket): the kernel's last CTA raises this
    rank's "partial ready" flag on every rank (b200dsa_sparse_mla_decode_signal).  pair=True runs the
    cluster-of-two kernel (b200dsa_sparse_mla_decode_pair: same results, measured slower)."""
    require_cuda(q, kv, indices, kv_row_base, q_pos)
    if q.dtype != torch.bfloat16 or not q.is_contiguous() or q.dim() != 3 or q.shape[2] != 576:
        raise _lib.B200DSAError("q must be contiguous bf16 [n_items, n_heads, 576]")
    if kv.dtype != torch.bfloat16 or not kv.is_contiguous() or kv.dim() != 2 or kv.shape[1] != 576:
        raise _lib.B200DSAError("kv must be contiguous bf16 [rows, 576]")
    if indices.dtype != torch.int32 or indices.dim() != 2 or indices.stride(1) != 1 or indices.shape[0] != q.shape[0]:
        raise _lib.B200DSAError("indices must be int32 [n_items, n_idx] with unit column stride")
    if kv_row_base is not None and (kv_row_base.dtype != torch.int64 or not kv_row_base.is_contiguous()):
        raise _lib.B200DSAError("kv_row_base must be contiguous int64")
    _i32(q_pos, "q_pos")
    n, H, _ = q.shape
    if ctx is None:
        ctx = torch.empty(n, H, 512, dtype=torch.float32, device=q.device)
    if lse is None:
        lse = torch.empty(n, H, dtype=torch.float32, device=q.device)
    if ctx.dtype not in (torch.float32, torch.bfloat16) or not ctx.is_contiguous() or ctx.shape != (n, H, 512):
        raise _lib.B200DSAError("ctx must be contiguous fp32 or bf16 [n_items, n_heads, 512]")
    lib = _lib.load()
    args = (ptr(q), ptr(kv), kv.shape[0], ptr(kv_row_base), ptr(indices), indices.stride(0), indices.shape[1],
            ptr(_i32(n_idx_item, "n_idx_item")), ptr(q_pos), q_pos_bias, pos_lo, pos_hi, n, H, sm_scale, ptr(ctx),
            int(ctx.dtype == torch.bfloat16), ptr(lse))
    if pair:
        if signal is not None:
            raise _lib.B200DSAError("the cluster-of-two kernel has no signalling form")
        rc = lib.b200dsa_sparse_mla_decode_pair(*args, ptr(status_word(q.device)), stream_ptr())
    elif signal is None:
        rc = lib.b200dsa_sparse_mla_decode(*args, ptr(status_word(q.device)), stream_ptr())
    else:
        link, ticket = signal
        rc = lib.b200dsa_sparse_mla_decode_signal(*args, ctypes.byref(link), ptr(ticket), ptr(status_word(q.device)),
                                                  stream_ptr())
    check(rc, "b200dsa_sparse_mla_decode")
    return ctx, lse


def topk_merge_owned(recv: torch.Tensor, k: int, own_lo: int, own_hi: int, *, out: torch.Tensor,
                     owned: torch.Tensor, owned_count: torch.Tensor, sorted: bool = False, link=None):
    """Global top-k of every row from the per-rank selections in recv int32 [world, n_rows, 2k]
    (positions, then score bit patterns), plus the winners inside [own_lo, own_hi) compacted into
    `owned`; see b200dsa_topk_merge_owned.  link: wait for the peers' pushes first."""
    require_cuda(recv, out, owned, owned_count)
    if recv.dtype != torch.int32 or not recv.is_contiguous() or recv.dim() != 3 or recv.shape[2] != 2 * k:
        raise _lib.B200DSAError("recv must be contiguous int32 [world, n_rows, 2k]")
    world, n_rows, _ = recv.shape
    _check_topk_outputs(out, None, n_rows, k)
    _check_topk_outputs(owned, None, n_rows, k)
    if _i32(owned_count, "owned_count").numel() < n_rows:
        raise _lib.B200DSAError("owned_count needs one entry per row")
    rc = _lib.load().b200dsa_topk_merge_owned(
        ptr(recv), world, n_rows, k, int(sorted), own_lo, own_hi, ptr(out), out.stride(0), ptr(owned),
        owned.stride(0), ptr(owned_count), ctypes.byref(link) if link is not None else None,
        ptr(status_word(recv.device)), stream_ptr())
    check(rc, "b200dsa_topk_merge_owned")
    return out[:n_rows, :k], owned, owned_count


def lse_combine(ctx_parts: torch.Tensor, lse_parts: torch.Tensor, *, ctx_out: Optional[torch.Tensor] = None,
                lse_out: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Merge partials [R, ..., 512] / [R, ...] over R disjoint key sets; see b200dsa_lse_combine."""
    require_cuda(ctx_parts, lse_parts)
    if ctx_parts.dtype != torch.float32 or lse_parts.dtype != torch.float32 or \
            not ctx_parts.is_contiguous() or not lse_parts.is_contiguous() or ctx_parts.shape[-1] != 512:
        raise _lib.B200DSAError("partials must be contiguous fp32 [R, ..., 512] and [R, ...]")
    R = ctx_parts.shape[0]
    n_rows = lse_parts[0].numel()
    if ctx_out is None:
        ctx_out = torch.empty(ctx_parts.shape[1:], dtype=torch.float32, device=ctx_parts.device)
    if lse_out is None:
        lse_out = torch.empty(lse_parts.shape[1:], dtype=torch.float32, device=ctx_parts.device)
    rc = _lib.load().b200dsa_lse_combine(ptr(ctx_parts), ptr(lse_parts), R, n_rows, ptr(ctx_out), ptr(lse_out),
                                         stream_ptr())
    check(rc, "b200dsa_lse_combine")
    return ctx_out, lse_out


def quant_q_fold_weights(q: torch.Tensor, w: torch.Tensor, fold: float, *, q_fp8: Optional[torch.Tensor] = None,
                         weights: Optional[torch.Tensor] = None, ue8m0: bool = False
                         ) -> Tuple[torch.Tensor, torch.Tensor]:
    """(q_fp8 [..., H, 128] e4m3, weights [..., H] fp32) with the per-(token, head) scale folded
    into the weights; see b200dsa_quant_q_fold_weights.  ue8m0=True rounds every scale up to a
    power of two (the reference's use_ue8m0=True)."""
    require_cuda(q, w)
    if q.dtype != torch.bfloat16 or not q.is_contiguous() or q.shape[-1] != 128:
        raise _lib.B200DSAError("q must be contiguous bf16 [..., 128]")
    n_rows = q.numel() // 128
    if w.dtype != torch.float32 or not w.is_contiguous() or w.numel() != n_rows:
        raise _lib.B200DSAError("w must be contiguous fp32 with one entry per (token, head)")
    if q_fp8 is None:
        q_fp8 = torch.empty(q.shape, dtype=torch.float8_e4m3fn, device=q.device)
    if weights is None:
        weights = torch.empty(w.shape, dtype=torch.float32, device=q.device)
    rc = _lib.load().b200dsa_quant_q_fold_weights(ptr(q), ptr(w), n_rows, fold, int(bool(ue8m0)), ptr(q_fp8),
                                                  ptr(weights), stream_ptr())
    check(rc, "b200dsa_quant_q_fold_weights")
    return q_fp8, weights


WIRE_ROW = 516  # floats per (item, head) row of the all-reduce wire buffer


def lse_prescale(ctx: torch.Tensor, lse: torch.Tensor, lse_max: torch.Tensor, wire: torch.Tensor) -> torch.Tensor:
    """wire[row] = (ctx*exp(lse-lse_max), exp(lse-lse_max), 0, 0, 0); see b200dsa_lse_prescale."""
    require_cuda(ctx, lse, lse_max, wire)
    n_rows = lse.numel()
    for t_, nm in ((ctx, "ctx"), (lse, "lse"), (lse_max, "lse_max"), (wire, "wire")):
        if t_.dtype != torch.float32 or not t_.is_contiguous():
            raise _lib.B200DSAError(f"{nm} must be contiguous fp32")
    if ctx.numel() != n_rows * 512 or wire.numel() != n_rows * WIRE_ROW:
        raise _lib.B200DSAError("ctx must hold 512 and wire 516 floats per row")
    check(_lib.load().b200dsa_lse_prescale(ptr(ctx), ptr(lse), ptr(lse_max), n_rows, ptr(wire), stream_ptr()),
          "b200dsa_lse_prescale")
    return wire


def lse_finalize(wire: torch.Tensor, lse_max: torch.Tensor, ctx_out: torch.Tensor, lse_out: torch.Tensor):
    """Divide the summed wire rows by the summed weight; see b200dsa_lse_finalize."""
    require_cuda(wire, lse_max, ctx_out, lse_out)
    n_rows = lse_max.numel()
    check(_lib.load().b200dsa_lse_finalize(ptr(wire), ptr(lse_max), n_rows, ptr(ctx_out), ptr(lse_out),
                                            stream_ptr()), "b200dsa_lse_finalize")
    return ctx_out, lse_out


def block_mean_pool(keys: torch.Tensor, block: int, *, want_f32: bool = False):
    """Pooled keys bf16 [ceil(n/block), 128] (and fp32 copy when want_f32); see
    b200dsa_block_mean_pool_bf16."""
    require_cuda(keys)
    if keys.dtype != torch.bfloat16 or not keys.is_contiguous() or keys.dim() != 2 or keys.shape[1] != 128:
        raise _lib.B200DSAError("keys must be contiguous bf16 [n, 128]")
    nb = (keys.shape[0] + block - 1) // block
    out = torch.empty(nb, 128, dtype=torch.bfloat16, device=keys.device)
    out32 = torch.empty(nb, 128, dtype=torch.float32, device=keys.device) if want_f32 else None
    check(_lib.load().b200dsa_block_mean_pool_bf16(ptr(keys), keys.shape[0], block, ptr(out), ptr(out32),
                                                  stream_ptr()), "b200dsa_block_mean_pool_bf16")
    return (out, out32) if want_f32 else out


def paged_mean_pool_fp8(cache: torch.Tensor, page_size: int, context_lens: torch.Tensor,
                        block_table: torch.Tensor, block: int, max_pool_blocks: int) -> torch.Tensor:
    """fp32 [n_requests, max_pool_blocks, 128] block means over the paged FP8 cache."""
    require_cuda(cache, context_lens, block_table)
    _i32(context_lens, "context_lens"); _i32(block_table, "block_table")
    num_pages = cache.numel() // (page_size * 132)
    B = context_lens.numel()
    out = torch.empty(B, max_pool_blocks, 128, dtype=torch.float32, device=cache.device)
    check(_lib.load().b200dsa_paged_mean_pool_fp8(ptr(cache), num_pages, page_size, ptr(context_lens),
                                                 ptr(block_table), block_table.stride(0), B, block, max_pool_blocks,
                                                 ptr(out), ptr(status_word(cache.device)), stream_ptr()),
          "b200dsa_paged_mean_pool_fp8")
    return out


class PooledKeyCache:
    """Block means of the paged FP8 index-key cache kept up to date across decode steps
    (b200dsa_paged_mean_pool_fp8_update): every update() reads only the keys a request gained since
    the previous one.  One slot per request row; reset(rows) marks slots whose request changed so
    that the next update rebuilds them from the cache.  means is fp32 [n_slots, max_pool_blocks, 128],
    bit-identical to paged_mean_pool_fp8 on the same cache, lengths and tables."""

    def __init__(self, n_slots: int, max_pool_blocks: int, block: int, device):
        self.block, self.max_pool_blocks = block, max_pool_blocks
        self.sums = torch.zeros(n_slots, max_pool_blocks, 128, dtype=torch.float32, device=device)
        self.means = torch.zeros_like(self.sums)
        self.lens = torch.zeros(n_slots, dtype=torch.int32, device=device)
        self._fresh = True

    def reset(self, rows: Optional[torch.Tensor] = None) -> None:
        if rows is None:
            self.lens.zero_()
        else:
            self.lens[rows.long()] = 0
        self._fresh = True

    def update(self, cache: torch.Tensor, page_size: int, context_lens: torch.Tensor,
               block_table: torch.Tensor) -> torch.Tensor:
        require_cuda(cache, context_lens, block_table)
        _i32(context_lens, "context_lens"); _i32(block_table, "block_table")
        B = context_lens.numel()
        if B != self.lens.numel():
            raise _lib.B200DSAError("one context length per slot")
        num_pages = cache.numel() // (page_size * 132)
        ctas = min(self.max_pool_blocks, 256) if self._fresh else 2
        check(_lib.load().b200dsa_paged_mean_pool_fp8_update(
            ptr(cache), num_pages, page_size, ptr(self.lens), ptr(context_lens), ptr(block_table),
            block_table.stride(0), B, self.block, self.max_pool_blocks, ctas, ptr(self.sums), ptr(self.means),
            ptr(status_word(cache.device)), stream_ptr()), "b200dsa_paged_mean_pool_fp8_update")
        self.lens.copy_(context_lens)
        self._fresh = False
        return self.means


def _router_out(n_tokens: int, n_keep: int, device):
    return (torch.empty(n_tokens, 64, dtype=torch.float32, device=device),
            torch.empty(n_tokens, n_keep, dtype=torch.int32, device=device))


def router_qnorm_topk(q: torch.Tensor, w: torch.Tensor, n_keep: int):
    """(weights [T,64] zero on dropped heads, head_idx int32 [T,n_keep]); see b200dsa_router_qnorm_topk."""
    require_cuda(q, w)
    if q.dtype != torch.bfloat16 or not q.is_contiguous() or q.shape[-2:] != (64, 128):
        raise _lib.B200DSAError("q must be contiguous bf16 [T, 64, 128]")
    T = q.numel() // (64 * 128)
    wo, hi = _router_out(T, n_keep, q.device)
    check(_lib.load().b200dsa_router_qnorm_topk(ptr(q), ptr(w.contiguous()), T, n_keep, ptr(wo), ptr(hi),
                                                stream_ptr()), "b200dsa_router_qnorm_topk")
    return wo, hi


def router_block_score_topk(q: torch.Tensor, w: torch.Tensor, pooled: torch.Tensor, blk_lo: torch.Tensor,
                            blk_hi: torch.Tensor, n_keep: int, *, pooled_set: Optional[torch.Tensor] = None,
                            return_scores: bool = False):
    """Block-score router; pooled fp32 [n_blocks,128] or [n_sets,n_blocks,128]."""
    require_cuda(q, w, pooled, blk_lo, blk_hi, pooled_set)
    if pooled.dtype != torch.float32 or not pooled.is_contiguous():
        raise _lib.B200DSAError("pooled keys must be contiguous fp32")
    T = q.numel() // (64 * 128)
    set_stride = pooled.shape[-2] * 128 if pooled.dim() == 3 else 0
    wo, hi = _router_out(T, n_keep, q.device)
    sc = torch.empty(T, 64, dtype=torch.float32, device=q.device) if return_scores else None
    check(_lib.load().b200dsa_router_block_score_topk(
        ptr(q), ptr(w.contiguous()), ptr(pooled), set_stride, ptr(_i32(pooled_set, "pooled_set")),
        ptr(_i32(blk_lo, "blk_lo")), ptr(_i32(blk_hi, "blk_hi")), T, n_keep, ptr(wo), ptr(hi), ptr(sc),
        stream_ptr()), "b200dsa_router_block_score_topk")
    return (wo, hi, sc) if return_scores else (wo, hi)


def router_linear_topk_softmax(x: torch.Tensor, w_r: torch.Tensor, n_keep: int, *, return_logits: bool = False,
                               out_scale: Optional[torch.Tensor] = None):
    """Linear router: top-n of x @ W_r with softmax weights over the kept heads; out_scale fp32 [T, 64]
    multiplies the weights written (the folded per-head query scales of the FP8 indexer)."""
    require_cuda(x, w_r, out_scale)
    if out_scale is not None and (out_scale.dtype != torch.float32 or not out_scale.is_contiguous() or
                                  out_scale.shape != (x.shape[0], 64)):
        raise _lib.B200DSAError("out_scale must be contiguous fp32 [T, 64]")
    if x.dtype != torch.bfloat16 or w_r.dtype != torch.bfloat16 or not x.is_contiguous() or \
            not w_r.is_contiguous() or w_r.shape != (x.shape[1], 64):
        raise _lib.B200DSAError("x must be bf16 [T, hidden] and W_r bf16 [hidden, 64], both contiguous")
    T, hidden = x.shape
    wo, hi = _router_out(T, n_keep, x.device)
    lg = torch.empty(T, 64, dtype=torch.float32, device=x.device) if return_logits else None
    check(_lib.load().b200dsa_router_linear_topk_softmax(ptr(x), ptr(w_r), T, hidden, n_keep, ptr(out_scale), ptr(wo),
                                                        ptr(hi), ptr(lg), stream_ptr()),
          "b200dsa_router_linear_topk_softmax")
    return (wo, hi, lg) if return_logits else (wo, hi)


def indexer_k_quant_and_cache(k: torch.Tensor, cache: torch.Tensor, slot_mapping: torch.Tensor,
                              page_size: int, scale_fmt: Optional[str] = None) -> None:
    """Quantise new index keys and write them into their cache slots; see
    b200dsa_indexer_k_quant_and_cache.  scale_fmt "ue8m0" stores power-of-two scales, None plain
    amax/448 scales; any other string is rejected."""
    if scale_fmt not in (None, "ue8m0"):
        raise _lib.B200DSAError(f"unknown scale_fmt {scale_fmt!r} (None or 'ue8m0')")
    require_cuda(k, cache, slot_mapping)
    if k.dtype != torch.bfloat16 or not k.is_contiguous() or k.shape[-1] != 128:
        raise _lib.B200DSAError("k must be contiguous bf16 [n, 128]")
    if slot_mapping.dtype != torch.int64 or not slot_mapping.is_contiguous():
        raise _lib.B200DSAError("slot_mapping must be contiguous int64")
    if cache.dtype != torch.uint8 or not cache.is_contiguous():
        raise _lib.B200DSAError("cache must be a contiguous uint8 tensor")
    n = slot_mapping.numel()
    num_pages = cache.numel() // (page_size * 132)
    check(_lib.load().b200dsa_indexer_k_quant_and_cache(ptr(k), ptr(slot_mapping), n, ptr(cache), num_pages,
                                                        page_size, int(scale_fmt == "ue8m0"),
                                                        ptr(status_word(k.device)), stream_ptr()),
          "b200dsa_indexer_k_quant_and_cache")


def compact_owned(indices: torch.Tensor, pos_lo: int, pos_hi: int, out: torch.Tensor, count: torch.Tensor):
    """Positions inside [pos_lo, pos_hi) first, -1 after, count per row; see b200dsa_compact_owned."""
    require_cuda(indices, out, count)
    n_rows, n_idx = indices.shape
    check(_lib.load().b200dsa_compact_owned(ptr(indices), indices.stride(0), n_rows, n_idx, pos_lo, pos_hi, ptr(out),
                                            out.stride(0), ptr(_i32(count, "count")), stream_ptr()),
          "b200dsa_compact_owned")
    return out, count


def lse_prescale_norm(ctx: torch.Tensor, lse_all: torch.Tensor, my_part: int, out_bf16: torch.Tensor,
                      lse_out: torch.Tensor):
    """This rank's normalised bf16 share of the merged context; see b200dsa_lse_prescale_norm."""
    require_cuda(ctx, lse_all, out_bf16, lse_out)
    n_parts = lse_all.shape[0]
    n_rows = lse_all[0].numel()
    if ctx.dtype != torch.float32 or lse_all.dtype != torch.float32 or out_bf16.dtype != torch.bfloat16 or \
            not (ctx.is_contiguous() and lse_all.is_contiguous() and out_bf16.is_contiguous()):
        raise _lib.B200DSAError("ctx / lse_all must be contiguous fp32 and out_bf16 contiguous bf16")
    check(_lib.load().b200dsa_lse_prescale_norm(ptr(ctx), ptr(lse_all), n_parts, my_part, n_rows, ptr(out_bf16),
                                                ptr(lse_out), stream_ptr()), "b200dsa_lse_prescale_norm")
    return out_bf16, lse_out


def mma_peak_tflops(fp8: bool = True, *, iters: int = 4096, reps: int = 5, device=None) -> float:
    """Best-of-`reps` tensor-pipe throughput (TFLOP/s, dense) of back-to-back M=128 x N=256 tcgen05
    MMAs on shared-memory operands, one CTA per SM; see b200dsa_mma_peak_probe.  Synchronises."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    ctas = torch.cuda.get_device_properties(dev).multi_processor_count
    lib = _lib.load()
    st = status_word(dev)
    best = 0.0
    for r in range(reps + 1):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        check(lib.b200dsa_mma_peak_probe(int(fp8), ctas, iters, ptr(st), stream_ptr()), "b200dsa_mma_peak_probe")
        e1.record()
        torch.cuda.synchronize()
        if r == 0:
            continue                                     # warm-up launch
        flops = ctas * iters * 8 * 2.0 * 128 * 256 * (32 if fp8 else 16)
        best = max(best, flops / (e0.elapsed_time(e1) * 1e-3) / 1e12)
    return best


def sparse_attn_bwd_pointwise(s: torch.Tensor, dp: torch.Tensor, lse: torch.Tensor, delta: torch.Tensor,
                              indices: torch.Tensor, q_pos: torch.Tensor, scale: float):
    """(p, ds) of the attention backward from raw scores s and dp [T, H, K] (bf16 or fp32, same dtype out);
    see b200dsa_sparse_attn_bwd_pointwise."""
    require_cuda(s, dp, lse, delta, indices, q_pos)
    if s.dtype not in (torch.bfloat16, torch.float32) or dp.dtype != s.dtype or s.shape != dp.shape or s.dim() != 3 or \
            not s.is_contiguous() or not dp.is_contiguous():
        raise _lib.B200DSAError("s and dp must be contiguous [T, H, K] of the same dtype (bf16 or fp32)")
    T, H, Kk = s.shape
    for t_, nm, shape in ((lse, "lse", (T, H)), (delta, "delta", (T, H))):
        if t_.dtype != torch.float32 or not t_.is_contiguous() or tuple(t_.shape) != shape:
            raise _lib.B200DSAError(f"{nm} must be contiguous fp32 [T, H]")
    if _i32(indices, "indices").shape != (T, Kk) or _i32(q_pos, "q_pos").numel() != T:
        raise _lib.B200DSAError("indices must be int32 [T, K] and q_pos int32 [T]")
    p, ds = torch.empty_like(s), torch.empty_like(s)
    check(_lib.load().b200dsa_sparse_attn_bwd_pointwise(ptr(s), ptr(dp), int(s.dtype == torch.bfloat16), ptr(lse),
                                                       ptr(delta), ptr(indices), ptr(q_pos), T, H, Kk, scale, ptr(p),
                                                       ptr(ds), stream_ptr()), "b200dsa_sparse_attn_bwd_pointwise")
    return p, ds


def scatter_add_latent_rows(d_latent: torch.Tensor, rows_qk: torch.Tensor, rows_v: Optional[torch.Tensor],
                            indices: torch.Tensor, q_pos: torch.Tensor) -> None:
    """d_latent[indices[t,j]] += rows_qk[t,j] (+ rows_v[t,j] on the first 512 columns) over the valid entries;
    see b200dsa_scatter_add_latent_rows."""
    require_cuda(d_latent, rows_qk, rows_v, indices, q_pos)
    if d_latent.dtype != torch.float32 or not d_latent.is_contiguous() or d_latent.shape[-1] != 576:
        raise _lib.B200DSAError("d_latent must be contiguous fp32 [rows, 576]")
    if rows_qk.dtype not in (torch.bfloat16, torch.float32) or not rows_qk.is_contiguous() or rows_qk.dim() != 3 or \
            rows_qk.shape[-1] != 576:
        raise _lib.B200DSAError("rows_qk must be contiguous [T, K, 576] bf16 or fp32")
    T, Kk = rows_qk.shape[:2]
    if rows_v is not None and (rows_v.dtype != rows_qk.dtype or not rows_v.is_contiguous() or
                               tuple(rows_v.shape) != (T, Kk, 512)):
        raise _lib.B200DSAError("rows_v must be contiguous [T, K, 512] of the dtype of rows_qk")
    if _i32(indices, "indices").shape != (T, Kk) or _i32(q_pos, "q_pos").numel() != T:
        raise _lib.B200DSAError("indices must be int32 [T, K] and q_pos int32 [T]")
    check(_lib.load().b200dsa_scatter_add_latent_rows(ptr(d_latent), d_latent.shape[0], ptr(rows_qk), ptr(rows_v),
                                                     int(rows_qk.dtype == torch.bfloat16), ptr(indices), ptr(q_pos), T,
                                                     Kk, ptr(status_word(d_latent.device)), stream_ptr()),
          "b200dsa_scatter_add_latent_rows")


def mma_shape_clocks(m: int, n: int, a_from_tmem: bool, *, iters: int = 2048, device=None) -> float:
    """SM clocks per bf16 tcgen05 MMA of shape m x n x 16 issued back to back, the A operand in shared or
    tensor memory (one CTA per SM, counted inside the kernel); see b200dsa_mma_shape_probe.  Synchronises."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    ctas = torch.cuda.get_device_properties(dev).multi_processor_count
    clocks = torch.zeros(ctas, dtype=torch.int64, device=dev)
    for _ in range(2):
        check(_lib.load().b200dsa_mma_shape_probe(m, n, int(a_from_tmem), ctas, iters, ptr(clocks),
                                                  ptr(status_word(dev)), stream_ptr()), "b200dsa_mma_shape_probe")
    torch.cuda.synchronize()
    return float(clocks.float().median()) / (iters * 4)


def hbm_read_gbs(buf: torch.Tensor, offsets: torch.Tensor, chunk_bytes: int, *, chunks_per_stage: int = 1,
                 ctas_per_sm: int = 2, reps: int = 10) -> float:
    """GB/s at which the chunks buf + offsets[i] (int64 byte offsets, chunk_bytes each) are read by bare bulk
    copies into a shared-memory ring; see b200dsa_hbm_read_probe.  Synchronises."""
    require_cuda(buf, offsets)
    if offsets.dtype != torch.int64 or not offsets.is_contiguous():
        raise _lib.B200DSAError("offsets must be contiguous int64")
    ctas = torch.cuda.get_device_properties(buf.device).multi_processor_count * ctas_per_sm
    n = offsets.numel() // chunks_per_stage * chunks_per_stage
    st = status_word(buf.device)

    def run():
        check(_lib.load().b200dsa_hbm_read_probe(ptr(buf), ptr(offsets), n, chunk_bytes, chunks_per_stage, ctas,
                                                 ptr(st), stream_ptr()), "b200dsa_hbm_read_probe")
    for _ in range(2):
        run()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        run()
    e1.record()
    torch.cuda.synchronize()
    return n * chunk_bytes * reps / (e0.elapsed_time(e1) * 1e-3) / 1e9


def _f32c(t: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    return None if t is None else t.to(torch.float32).contiguous()


def indexer_k_norm_rope(k_proj: torch.Tensor, ln_weight: Optional[torch.Tensor], ln_bias: Optional[torch.Tensor],
                        eps: float, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], *,
                        rope_first: bool = False, want_rows: bool = True, cache: Optional[torch.Tensor] = None,
                        slot_mapping: Optional[torch.Tensor] = None, page_size: int = 64,
                        scale_fmt: Optional[str] = None) -> Optional[torch.Tensor]:
    """k = RoPE(LayerNorm(k_proj)) for rows [n_tokens, 128] (bf16 or fp32); see b200dsa_indexer_k_norm_rope.
    Returns the rows (input dtype) unless want_rows=False; with `cache` + `slot_mapping` the rows are also
    quantised and written into their cache slots in the same kernel."""
    require_cuda(k_proj, ln_weight, ln_bias, cos, sin, cache, slot_mapping)
    if k_proj.dtype not in (torch.bfloat16, torch.float32) or not k_proj.is_contiguous() or k_proj.shape[-1] != 128:
        raise _lib.B200DSAError("k_proj must be contiguous bf16 or fp32 [..., 128]")
    if scale_fmt not in (None, "ue8m0"):
        raise _lib.B200DSAError(f"unknown scale_fmt {scale_fmt!r} (None or 'ue8m0')")
    n = k_proj.numel() // 128
    lw, lb, c, s_ = _f32c(ln_weight), _f32c(ln_bias), _f32c(cos), _f32c(sin)
    if c is not None and (c.numel() != n * 64 or s_.numel() != n * 64):
        raise _lib.B200DSAError("cos / sin must hold 64 values per token")
    out = torch.empty_like(k_proj) if want_rows else None
    num_pages = 0
    if cache is not None:
        if cache.dtype != torch.uint8 or not cache.is_contiguous() or slot_mapping is None or \
                slot_mapping.dtype != torch.int64 or slot_mapping.numel() != n:
            raise _lib.B200DSAError("cache must be contiguous uint8 and slot_mapping int64 with one entry per token")
        num_pages = cache.numel() // (page_size * 132)
    rc = _lib.load().b200dsa_indexer_k_norm_rope(
        ptr(k_proj), int(k_proj.dtype == torch.float32), n, ptr(lw), ptr(lb), eps, ptr(c), ptr(s_), int(rope_first),
        ptr(out), ptr(slot_mapping), ptr(cache), num_pages, page_size, int(scale_fmt == "ue8m0"),
        ptr(status_word(k_proj.device)), stream_ptr())
    check(rc, "b200dsa_indexer_k_norm_rope")
    return out


def indexer_q_rope(q_proj: torch.Tensor, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], *,
                   rope_first: bool = False, want_rows: bool = True, w: Optional[torch.Tensor] = None,
                   fold: float = 1.0, ue8m0: bool = False):
    """RoPE on the rows of q_proj [n_tokens, n_heads, 128] (bf16 or fp32); see b200dsa_indexer_q_rope.
    Returns the rows, or with `w` [n_tokens, n_heads] (rows, q_fp8, weights) / (q_fp8, weights): the FP8
    quantisation with the scale folded into the head weights, from the same kernel."""
    require_cuda(q_proj, cos, sin, w)
    if q_proj.dtype not in (torch.bfloat16, torch.float32) or not q_proj.is_contiguous() or q_proj.dim() != 3 or \
            q_proj.shape[-1] != 128:
        raise _lib.B200DSAError("q_proj must be contiguous bf16 or fp32 [n_tokens, n_heads, 128]")
    T, H, _ = q_proj.shape
    c, s_ = _f32c(cos), _f32c(sin)
    if c is not None and (c.numel() != T * 64 or s_.numel() != T * 64):
        raise _lib.B200DSAError("cos / sin must hold 64 values per token")
    out = torch.empty_like(q_proj) if want_rows else None
    q_fp8 = weights = wc = None
    if w is not None:
        wc = w.to(torch.float32).contiguous()
        if wc.numel() != T * H:
            raise _lib.B200DSAError("w must hold one weight per (token, head)")
        q_fp8 = torch.empty(T, H, 128, dtype=torch.float8_e4m3fn, device=q_proj.device)
        weights = torch.empty(T, H, dtype=torch.float32, device=q_proj.device)
    rc = _lib.load().b200dsa_indexer_q_rope(
        ptr(q_proj), int(q_proj.dtype == torch.float32), T, H, ptr(c), ptr(s_), int(rope_first), ptr(out), ptr(wc),
        fold, int(bool(ue8m0)), ptr(q_fp8), ptr(weights), stream_ptr())
    check(rc, "b200dsa_indexer_q_rope")
    if w is None:
        return out
    return (out, q_fp8, weights) if want_rows else (q_fp8, weights)


def wuv_up_project(ctx: torch.Tensor, w_uv: torch.Tensor, *, out_dtype: torch.dtype = torch.bfloat16,
                   out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t,h,:] = ctx[t,h,:] @ W_UV[h]^T: ctx bf16 [T, H, 512], W_UV bf16 [H, Dv, 512] -> [T, H, Dv];
    see b200dsa_wuv_up_project."""
    require_cuda(ctx, w_uv, out)
    if ctx.dtype != torch.bfloat16 or not ctx.is_contiguous() or ctx.dim() != 3 or ctx.shape[2] != 512:
        raise _lib.B200DSAError("ctx must be contiguous bf16 [n_tokens, n_heads, 512]")
    T, H, _ = ctx.shape
    if w_uv.dtype != torch.bfloat16 or not w_uv.is_contiguous() or w_uv.dim() != 3 or w_uv.shape[0] != H or \
            w_uv.shape[2] != 512 or not 1 <= w_uv.shape[1] <= 256:
        raise _lib.B200DSAError("W_UV must be contiguous bf16 [n_heads, dv <= 256, 512]")
    dv = w_uv.shape[1]
    if out is None:
        out = torch.empty(T, H, dv, dtype=out_dtype, device=ctx.device)
    if out.dtype not in (torch.bfloat16, torch.float32) or not out.is_contiguous() or out.shape != (T, H, dv):
        raise _lib.B200DSAError("out must be contiguous bf16 or fp32 [n_tokens, n_heads, dv]")
    rc = _lib.load().b200dsa_wuv_up_project(ptr(ctx), ptr(w_uv), T, H, dv, ptr(out), int(out.dtype == torch.float32),
                                            ptr(status_word(ctx.device)), stream_ptr())
    check(rc, "b200dsa_wuv_up_project")
    return out
