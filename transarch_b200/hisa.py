"""HISA two-stage selection (hierarchical indexed sparse attention):

    stage 1  pool the index keys into blocks of 128 (mean, tail-aware), score every block with
             the indexer formula, mask to the query's block range, force-keep the last
             (optionally also the first) valid block, keep the top-m blocks;
    stage 2  score tokens only inside the kept blocks, mask to [ks, ke), keep the top-k.

The TransArch repository describes HISA (HISA_COLM_2026/README.md:5-12, :41-47: block size
128, top-64 blocks) but ships no code for it; the pieces this follows are the TileLang
fragments in MISA_preprint/misa_vllm_patch_2stage/misa_vllm_patch/block_ops.py: mean pooling
(:685-754), block-sparse token logits (:756-937) and the clean / force-maintain masks
(:576-666).  Both stages run on the tcgen05 block-list indexer kernel: stage 1 treats the
pooled keys as the key tensor.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from . import kernels as K
from ._lib import B200DSAError
from .opendsa_ops import _pad_heads


@dataclass
class HisaConfig:
    """Names follow the external HISA configs (HISA_COLM_2026/README.md:41-47)."""
    use_hisa: bool = True
    hisa_k_block_size: int = 128
    hisa_block_topk: int = 64
    index_topk: int = 2048
    keep_first_block: bool = False   # block_ops.py:576-666 force-keeps the first and the last valid block;
    keep_last_block: bool = True     # the default here keeps only the last (the query's own block)


@torch.no_grad()
def hisa_block_logits(q: torch.Tensor, k_pooled: torch.Tensor, w: torch.Tensor, ks: torch.Tensor, ke: torch.Tensor,
                      cfg: HisaConfig, sm_scale: float) -> torch.Tensor:
    """Stage-1 block scores fp32 [T, 128*ceil(n_blocks/128)]: the indexer formula on the pooled keys,
    -inf outside the query's block range [ks // P, ceil(ke / P)), +inf on the force-kept blocks (what
    the reference's clean_and_maintain_logits_ fragment does to a block-score matrix,
    block_ops.py:636-666)."""
    P = cfg.hisa_k_block_size
    T = q.shape[0]
    nb = k_pooled.shape[0]
    nb128 = (nb + 127) // 128
    dev = q.device
    bks = (ks // P).to(torch.int32).contiguous()
    bke = ((ke + P - 1) // P).to(torch.int32).clamp(max=nb).contiguous()
    # the pooled keys are a flat key tensor: the prefill kernel shares every tile of them between four
    # queries.  Its columns start at the tile of the lower bound, so the walk starts at block 0 (column =
    # block id) and the lower bound is masked afterwards.
    row_cols = (((bke + 127) >> 7) << 7).contiguous()
    logits = K.indexer_flat_bf16_logits(q, w, k_pooled, torch.zeros_like(bks), bke, row_cols, nb128 * 128,
                                        out_scale=sm_scale)
    cols = torch.arange(nb128 * 128, dtype=torch.int32, device=dev).view(1, -1)
    logits.masked_fill_(cols < bks.view(-1, 1), float("-inf"))
    # force-keep by a +inf score; rows without any valid block keep what they have (no host
    # synchronisation: a scatter of either +inf or the value already there)
    has = (bke > bks).view(-1, 1)
    inf = torch.full((T, 1), float("inf"), device=dev)
    if cfg.keep_last_block:
        col = (bke - 1).clamp(min=0).long().view(-1, 1)
        logits.scatter_(1, col, torch.where(has, inf, logits.gather(1, col)))
    if cfg.keep_first_block:
        col = bks.clamp(max=logits.shape[1] - 1).long().view(-1, 1)
        logits.scatter_(1, col, torch.where(has, inf, logits.gather(1, col)))
    return logits


@torch.no_grad()
def hisa_block_topk(q: torch.Tensor, k_pooled: torch.Tensor, w: torch.Tensor, ks: torch.Tensor, ke: torch.Tensor,
                    cfg: HisaConfig, sm_scale: float) -> torch.Tensor:
    """Stage 1: int32 [T, m] ids of the kept key blocks, best first, -1 padded."""
    logits = hisa_block_logits(q, k_pooled, w, ks, ke, cfg, sm_scale)
    return K.topk_select(logits, cfg.hisa_block_topk, keep_pos_inf=True, sorted=True)


@torch.no_grad()
def hisa_select_topk(index_q, index_k, index_w, ks, ke, cfg: Optional[HisaConfig] = None, *,
                     sm_scale_index: Optional[float] = None, return_blocks: bool = False):
    """Top-k key positions per query through the two-stage HISA path; int32 [T, index_topk],
    absolute positions, descending stage-2 score, -1 padded.  ks / ke are the per-query causal
    intervals (as prepare_ks_ke returns them)."""
    cfg = cfg or HisaConfig()
    if cfg.hisa_k_block_size != 128:
        raise B200DSAError("hisa_k_block_size must be 128 (one block per tensor-core key tile)")
    if not index_q.is_cuda:
        raise B200DSAError("hisa_select_topk needs CUDA tensors (no CPU path)")
    d = index_q.shape[-1]
    sf = sm_scale_index if sm_scale_index is not None else d ** -0.5
    q, w = _pad_heads(index_q.to(torch.bfloat16), index_w.to(torch.float32))
    k = index_k.to(torch.bfloat16).contiguous()
    k_pooled = K.block_mean_pool(k, cfg.hisa_k_block_size)
    blocks = hisa_block_topk(q, k_pooled, w, ks, ke, cfg, sf)
    n_blk = (blocks >= 0).sum(dim=1).to(torch.int32)
    row_cols = (n_blk * 128).contiguous()
    logits = K.indexer_blocklist_bf16_logits(q, w, k, blocks, row_cols, pos_lo=ks.to(torch.int32).contiguous(),
                                             pos_hi=ke.to(torch.int32).contiguous(), out_scale=sf)
    idx = K.topk_select(logits, cfg.index_topk, col_end=row_cols, page_table=blocks, page_size=128, sorted=True)
    return (idx, blocks) if return_blocks else idx


@torch.no_grad()
def hisa_select_topk_paged(q_fp8: torch.Tensor, weights: torch.Tensor, cache: torch.Tensor, page_size: int,
                           context_lens: torch.Tensor, block_table: torch.Tensor, cfg: Optional[HisaConfig] = None,
                           *, next_n: int = 1, max_model_len: Optional[int] = None, return_blocks: bool = False,
                           pooled: Optional[torch.Tensor] = None):
    """The two-stage HISA selection over the paged FP8 index-key cache (the serving layout): decode rows
    score the block means of their request, keep the top-m 128-key blocks (the last one always), then score
    tokens only inside those blocks, reading the FP8 pages in place.

      q_fp8 [rows, 64, 128] e4m3 and weights [rows, 64] fp32 (query scale folded in), rows = requests * next_n
      cache uint8 [num_pages, page_size*132], context_lens int32 [rows] (keys visible to each row),
      block_table int32 [requests, max_pages]
    Returns int32 [rows, index_topk] key positions inside the request (descending score, -1 padded).
    Stage 2 follows the reference's paged block-sparse fragment (block_ops.py:151-379); pooling is its
    paged_mean_pooling (:381-486).  pooled: the block means fp32 [requests, max_pool, 128] (max_pool =
    ceil(max_model_len / 128) rounded up to 128) from a kernels.PooledKeyCache that follows the cache,
    instead of pooling the whole cache in this call."""
    cfg = cfg or HisaConfig()
    if cfg.hisa_k_block_size != 128:
        raise B200DSAError("hisa_k_block_size must be 128 (one block per tensor-core key tile)")
    rows = q_fp8.shape[0]
    n_req = rows // next_n
    ctx = context_lens.to(torch.int32).contiguous()
    dev = q_fp8.device
    if max_model_len is None:
        max_model_len = block_table.shape[1] * page_size
    max_pool = ((max_model_len + 127) // 128 + 127) // 128 * 128         # pooled blocks per request, whole tiles
    req_ctx = ctx.view(n_req, next_n).max(dim=1).values.contiguous()
    if pooled is None:
        pooled = K.paged_mean_pool_fp8(cache, page_size, req_ctx, block_table, 128, max_pool)
    elif pooled.shape != (n_req, max_pool, 128) or pooled.dtype != torch.float32 or not pooled.is_contiguous():
        raise B200DSAError("pooled must be contiguous fp32 [requests, max_pool, 128]")
    k_pooled = pooled.view(n_req * max_pool, 128).to(torch.bfloat16)
    w = weights.to(torch.float32).contiguous()
    qb = q_fp8.to(torch.bfloat16).contiguous()
    # stage 1: row r reads the pooled set of its request (tiles req*max_pool/128 ...), block range [0, ceil(ctx/128))
    req = torch.arange(rows, device=dev, dtype=torch.int32) // next_n
    tiles = max_pool // 128
    lists = (req.view(-1, 1) * tiles + torch.arange(tiles, device=dev, dtype=torch.int32).view(1, -1)).contiguous()
    row_cols = torch.full((rows,), max_pool, dtype=torch.int32, device=dev)
    base = req * max_pool
    n_blk_ctx = (ctx + 127) // 128
    logits = K.indexer_blocklist_bf16_logits(qb, w, k_pooled, lists, row_cols, pos_lo=base.contiguous(),
                                             pos_hi=(base + n_blk_ctx).contiguous())
    has = (n_blk_ctx > 0).view(-1, 1)
    inf = torch.full((rows, 1), float("inf"), device=dev)
    if cfg.keep_last_block:
        col = (n_blk_ctx - 1).clamp(min=0).long().view(-1, 1)
        logits.scatter_(1, col, torch.where(has, inf, logits.gather(1, col)))
    if cfg.keep_first_block:
        col = torch.zeros(rows, 1, dtype=torch.long, device=dev)
        logits.scatter_(1, col, torch.where(has, inf, logits.gather(1, col)))
    blocks = K.topk_select(logits, cfg.hisa_block_topk, keep_pos_inf=True, sorted=True)
    # stage 2: tokens inside the kept blocks, straight from the FP8 pages
    n_blk = (blocks >= 0).sum(dim=1).to(torch.int32)
    tok_cols = (n_blk * 128).contiguous()
    tok = K.indexer_paged_blocklist_fp8_logits(q_fp8, w, cache, page_size, ctx, block_table, blocks, tok_cols,
                                               next_n=next_n)
    idx = K.topk_select(tok, cfg.index_topk, col_end=tok_cols, page_table=blocks, page_size=128, sorted=True)
    return (idx, blocks) if return_blocks else idx
