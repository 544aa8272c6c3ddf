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
    lists = torch.arange(nb128, dtype=torch.int32, device=dev).view(1, -1).expand(T, -1).contiguous()
    row_cols = torch.full((T,), nb128 * 128, dtype=torch.int32, device=dev)
    bks = (ks // P).to(torch.int32).contiguous()
    bke = ((ke + P - 1) // P).to(torch.int32).clamp(max=nb).contiguous()
    logits = K.indexer_blocklist_bf16_logits(q, w, k_pooled, lists, row_cols, pos_lo=bks, pos_hi=bke,
                                             out_scale=sm_scale)
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
