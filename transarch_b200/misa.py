"""MISA (mixture of indexer heads): a router keeps n of the 64 index heads per query, the
kept heads pick stage-1 candidates, all heads re-score the candidates.

Same names, arguments and tuple returns as the reference's orchestration functions:

    misa_mqa_logits       MISA_preprint/misa_vllm_patch_2stage/misa_vllm_patch/misa_ops.py:653-713
    misa_page_mqa_logits  MISA_preprint/misa_vllm_patch_2stage/misa_vllm_patch/misa_ops.py:344-413

Head gating is a zero weight on the dropped heads (it removes a head from the sum exactly).
The 64-head tensor-core kernels take the kept heads as a bit mask and write, in ONE pass over
the keys, both the routed stage-1 score and the all-head score that the reference computes in
a second pass over the candidates; stage 2 is then a gather.  The decode path reads the FP8
cache in place (the reference dequantises the whole cache to bf16 first, misa_ops.py:360-378).  Weights stay fp32 (the reference rounds them to
bf16 at :690); scores therefore follow the fp32-weight oracle.

Routers: q-norm (misa_deepseek_v2.py:254-266), block-score (block_ops.py:11-98, :488-573) and a
linear router x @ W_r with softmax weights over the kept heads (no reference code).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from . import kernels as K
from ._lib import B200DSAError
from .opendsa_ops import identity_block_lists


@dataclass
class MisaConfig:
    """HF config keys of the reference (MISA_preprint/README.md:44-62, read at
    misa_deepseek_v2.py:134-146)."""
    use_misa: bool = True
    misa_topk_heads: int = 8
    misa_decode_topk_heads: int = 8
    misa_k_block_size: int = 1024
    misa_use_qnorm: bool = False
    misa_stage1_topk: int = 8192
    index_topk: int = 2048
    index_n_heads: int = 64
    index_head_dim: int = 128


def gate_weights_by_heads(weights: torch.Tensor, head_idx: torch.Tensor) -> torch.Tensor:
    """Dense [M,64] weights that are zero except on head_idx (original weights kept there;
    misa_ops.py:703-705)."""
    out = torch.zeros_like(weights)
    idx = head_idx.long()
    return out.scatter_(1, idx, torch.gather(weights, 1, idx))


def _dequant_flat_keys(kv) -> torch.Tensor:
    k_fp8, k_scales = kv
    sc = k_scales.contiguous().view(torch.float32).reshape(-1, 1)
    return (k_fp8.float() * sc).to(torch.bfloat16).contiguous()        # misa_ops.py:682-690


@torch.no_grad()
def misa_mqa_logits(q: torch.Tensor, kv: Tuple[torch.Tensor, torch.Tensor], weights: torch.Tensor,
                    q_head_topk_indices: Optional[torch.Tensor], cu_seqlen_ks: torch.Tensor,
                    cu_seqlen_ke: torch.Tensor, use_qnorm: bool, topk_heads: int, stage1_topk: int,
                    k_block_size: Optional[int] = None):
    """Routed prefill logits over flat FP8 keys.  Returns (logits fp32 [M, s1] of all heads on the
    stage-1 candidates, sparse_topk_indices int32 [M, s1] key positions; -1 / -inf where a
    query sees fewer than s1 keys)."""
    k = _dequant_flat_keys(kv)
    qb = q.to(torch.bfloat16).contiguous()
    w = weights.to(torch.float32).contiguous()
    ks = cu_seqlen_ks.to(torch.int32).contiguous()
    ke = cu_seqlen_ke.to(torch.int32).contiguous()
    N = k.shape[0]
    if use_qnorm:
        if q_head_topk_indices is None:
            raise B200DSAError("use_qnorm needs q_head_topk_indices")
        head_idx = q_head_topk_indices[:, :topk_heads]
    else:
        if k_block_size is None:
            raise B200DSAError("k_block_size must be provided for the block-score router")
        _, pooled = K.block_mean_pool(k, k_block_size, want_f32=True)
        pooled = pooled.to(torch.bfloat16).float().contiguous()            # the reference pools to bf16
        _, head_idx = K.router_block_score_topk(qb, w, pooled, (ks // k_block_size).contiguous(),
                                                ((ke + k_block_size - 1) // k_block_size).contiguous(), topk_heads)
    s1 = min(stage1_topk, N)
    if head_idx.shape[1] <= 8 and N >= 2 * s1:
        return _misa_prefill_two_stage(qb, w, k, head_idx, ks, ke, s1)
    # short key ranges: one pass writes the routed and the all-head score of every key, stage 2 is a gather
    bl, row_cols = identity_block_lists(ks.long(), ke.long(), N)
    full, stage1 = K.indexer_blocklist_bf16_logits(qb, w, k, bl, row_cols, pos_lo=ks, pos_hi=ke,
                                                   head_mask=K.head_mask_from_indices(head_idx))
    cand = K.topk_select(stage1, s1, col_end=row_cols, page_table=bl, page_size=128, sorted=False)
    # candidate positions -> columns of `full` (column = position - 128*first block of the row)
    col0 = ((ks // 128) * 128).view(-1, 1)
    cols = (cand - col0).clamp(min=0).long()
    logits = torch.gather(full, 1, cols)
    logits = torch.where(cand >= 0, logits, torch.full_like(logits, float("-inf")))
    return logits, cand


_STAGE1_BYTES = 1 << 30     # bound on the routed score matrix of one query chunk


def _misa_prefill_two_stage(qb, w, k, head_idx, ks, ke, s1):
    """Long key ranges, where the routing saves work (misa_ops.py:415-515 stage 1 on the kept heads with
    block_Q = 128 / H queries per tile, :517-650 stage 2 on all heads over the candidates): the kept heads
    of every query are gathered into [M, 8, 128] and scored 32 queries per key tile; the top-s1 positions
    of that score are then re-scored with all 64 heads by the gathering kernel, 128 candidates per pass.
    Fewer than eight kept heads are padded with zero-weight copies."""
    M, N = qb.shape[0], k.shape[0]
    idx = head_idx.long()
    w8 = torch.gather(w, 1, idx)
    if idx.shape[1] < 8:
        pad = 8 - idx.shape[1]
        idx = torch.cat([idx, idx[:, :1].expand(-1, pad)], dim=1)
        w8 = torch.cat([w8, w8.new_zeros(M, pad)], dim=1)
    q8 = torch.gather(qb, 1, idx.view(M, 8, 1).expand(-1, -1, 128)).contiguous()
    w8 = w8.contiguous()
    col0 = ((ks >> 7) << 7).contiguous()
    row_cols = ((((ke + 127) >> 7) << 7) - col0).clamp_(min=0).contiguous()
    cols = ((N + 127) // 128) * 128
    cand = torch.empty(M, s1, dtype=torch.int32, device=qb.device)
    chunk = max(32, min(M, (_STAGE1_BYTES // (4 * cols)) // 32 * 32))
    buf = torch.empty(min(chunk, M), cols, dtype=torch.float32, device=qb.device)   # only columns < row_cols are read
    for t0 in range(0, M, chunk):
        t1 = min(M, t0 + chunk)
        stage1 = K.indexer_flat_bf16_logits_routed(q8[t0:t1], w8[t0:t1], k, ks[t0:t1], ke[t0:t1], row_cols[t0:t1], cols,
                                                   out=buf[:t1 - t0])
        K.topk_select(stage1[:t1 - t0], s1, col_end=row_cols[t0:t1], row_pos_offset=col0[t0:t1], sorted=False,
                      out=cand[t0:t1])
    logits = K.indexer_gather_bf16_logits(qb, w, k, cand, pos_lo=ks, pos_hi=ke)
    return logits, cand


@torch.no_grad()
def misa_page_mqa_logits(q_fp8: torch.Tensor, kv_cache_fp8: torch.Tensor, weights: torch.Tensor,
                         q_head_topk_indices: Optional[torch.Tensor], context_lens: torch.Tensor,
                         block_tables: torch.Tensor, max_model_len: int, decode_topk_heads: int, use_qnorm: bool,
                         stage1_topk: int, k_block_size: Optional[int] = None, *,
                         pooled: Optional[torch.Tensor] = None):
    """Routed decode logits over the paged FP8 cache.  q_fp8 [B, next_n, 64, 128] e4m3,
    kv_cache_fp8 uint8 [num_blocks, block_size, 1, 132] (or any view of those bytes), weights
    fp32 [B*next_n, 64].  Returns (logits [B*next_n, s1], sparse_topk_indices int32 [B*next_n, s1]).
    pooled (not in the reference's signature): block means fp32 [B, ceil(max_model_len / k_block_size), 128]
    kept up to date by kernels.PooledKeyCache, instead of pooling the whole cache again on every call."""
    B, next_n = q_fp8.shape[0], q_fp8.shape[1]
    page_size = kv_cache_fp8.shape[1]
    cache = kv_cache_fp8.reshape(kv_cache_fp8.shape[0], -1)
    if cache.dtype != torch.uint8:
        cache = cache.view(torch.uint8)
    cache = cache.contiguous()
    rows = B * next_n
    w = weights.to(torch.float32).reshape(rows, 64).contiguous()
    ctx = context_lens.to(torch.int32).contiguous()
    # row (b, n) sees context_lens[b] - next_n + n + 1 keys (indexers.py:545-551)
    n_off = torch.arange(next_n, device=ctx.device, dtype=torch.int32)
    row_ctx = (ctx.view(-1, 1) - next_n + n_off.view(1, -1) + 1).clamp(min=0).reshape(-1).contiguous()
    tables = block_tables.to(torch.int32).contiguous()
    if use_qnorm:
        if q_head_topk_indices is None:
            raise B200DSAError("use_qnorm needs q_head_topk_indices")
        head_idx = q_head_topk_indices.reshape(rows, -1)[:, :decode_topk_heads]
    else:
        if k_block_size is None:
            raise B200DSAError("k_block_size must be provided for the block-score router")
        max_pool = (max_model_len + k_block_size - 1) // k_block_size
        if pooled is None:
            pooled = K.paged_mean_pool_fp8(cache, page_size, ctx, tables, k_block_size, max_pool)
        elif pooled.shape != (B, max_pool, 128) or pooled.dtype != torch.float32 or not pooled.is_contiguous():
            raise B200DSAError("pooled must be contiguous fp32 [B, ceil(max_model_len / k_block_size), 128]")
        n_pool = ((row_ctx + k_block_size - 1) // k_block_size).to(torch.int32).contiguous()
        req = torch.arange(rows, device=ctx.device, dtype=torch.int32) // next_n
        qb = q_fp8.to(torch.bfloat16).reshape(rows, 64, 128).contiguous()
        _, head_idx = K.router_block_score_topk(qb, w, pooled, torch.zeros_like(n_pool), n_pool, decode_topk_heads,
                                                pooled_set=req.contiguous())
    q2 = q_fp8.reshape(rows, 64, 128).contiguous()
    s1 = min(stage1_topk, max_model_len)
    # columns beyond a row's context are never read below (col_end / valid candidates only): no fill
    full, stage1 = K.indexer_paged_fp8_logits(q2, w, cache, page_size, row_ctx, tables, next_n=next_n,
                                              max_cols=max_model_len, fill=False,
                                              head_mask=K.head_mask_from_indices(head_idx))
    cand = K.topk_select(stage1, s1, col_end=row_ctx, sorted=False)
    logits = torch.gather(full, 1, cand.clamp(min=0).long())
    logits = torch.where(cand >= 0, logits, torch.full_like(logits, float("-inf")))
    return logits, cand


@torch.no_grad()
def misa_final_topk(logits: torch.Tensor, sparse_topk_indices: torch.Tensor, topk_tokens: int,
                    out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Top-k of the stage-2 logits mapped back to key positions (indexers.py:499-504, :566-567)."""
    return K.topk_select(logits, min(topk_tokens, logits.shape[1]), pos_map=sparse_topk_indices.contiguous(),
                         sorted=True, out=out)


@torch.no_grad()
def misa_linear_router_decode(x: torch.Tensor, w_r: torch.Tensor, q_fp8: torch.Tensor, q_scale_fold: torch.Tensor,
                              cache: torch.Tensor, page_size: int, context_lens: torch.Tensor,
                              block_table: torch.Tensor, n_keep: int, topk: int, max_cols: Optional[int] = None):
    """Linear-router variant: logits = x @ W_r, keep the top-n heads, their softmax weights
    replace the head weights (times q_scale_fold [B,64], the per-head FP8 scale and softmax scale
    of the quantised queries), then indexer + top-k.  Returns (indices int32 [B, topk], head_idx)."""
    weights, head_idx = K.router_linear_topk_softmax(x.contiguous(), w_r.contiguous(), n_keep,
                                                     out_scale=q_scale_fold.to(torch.float32).contiguous())
    n_rows = q_fp8.numel() // (64 * 128)
    if topk <= 2048:
        # candidates collected by the indexer's own epilogue, one selection launch, logits kept only as the
        # exact fallback of a row whose list cannot be proven complete
        idx = K.indexer_paged_fp8_topk(q_fp8, weights, cache, page_size, context_lens, block_table, topk,
                                       K.fused_scratch_cached(n_rows, q_fp8.device), max_cols=max_cols, sorted=True)
        return idx, head_idx
    logits = K.indexer_paged_fp8_logits(q_fp8, weights, cache, page_size, context_lens, block_table,
                                        max_cols=max_cols, fill=False)
    if logits.shape[0] <= 148 and logits.shape[1] >= 32768 and topk <= 4096:
        # few long rows: several CTAs per row
        idx = K.topk_select_split(logits, topk, K.topk_scratch_cached(logits.shape[0], logits.device),
                                  col_end=context_lens, sorted=True)
    else:
        idx = K.topk_select(logits, topk, col_end=context_lens, sorted=True)
    return idx, head_idx
