"""Indexer-backend hook with the reference's vLLM signatures.

    MiSASparseAttnIndexer.forward_cuda(hidden_states, q_fp8, k, weights, q_head_topk_indices)
        MISA_preprint/misa_vllm_patch_2stage/misa_vllm_patch/indexers.py:628-712
    misa_sparse_attn_indexer(...)   same file :388-581 (the custom op it wraps)
    BaselineSparseAttnIndexer       same file :333-354 (dense DSA twin, no head routing)

What the op does per step: insert the new index keys into the paged FP8 cache, fill
topk_indices_buffer with -1, then for prefill chunks and for decode rows score the cached keys
and write each token's top-k key positions *relative to its request's first key* (int32, -1
padded) into its row of the buffer.  The buffer object itself is always returned (the
reference returns None on prefill-only steps, indexers.py:581).

Metadata: vLLM hands the op a per-layer metadata object through its forward context.  The
fields read here are the ones the reference reads (indexers.py:443-446, :474-495, :521-565);
any object with these attributes works, and the small dataclasses below can be filled
directly by tests or by an adapter for another vLLM version.  When `attn_metadata` is not
passed and vLLM is importable, it is taken from vllm.forward_context as the reference does.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

import torch

from . import kernels as K
from . import misa as M
from ._lib import B200DSAError


@dataclass
class PrefillChunk:
    token_start: int
    token_end: int
    block_table: torch.Tensor        # int32 [n_requests_in_chunk, max_blocks]
    cu_seq_lens: torch.Tensor        # int32 [n_requests_in_chunk + 1] key offsets of each request
    cu_seqlen_ks: torch.Tensor       # int32 [tokens] first visible key (offset into the chunk's keys)
    cu_seqlen_ke: torch.Tensor       # int32 [tokens] one past the last visible key
    total_seq_lens: int = 0


@dataclass
class PrefillMetadata:
    chunks: List[PrefillChunk] = field(default_factory=list)


@dataclass
class DecodeMetadata:
    seq_lens: torch.Tensor           # int32 [B]
    block_table: torch.Tensor        # int32 [B, max_blocks]
    decode_lens: Optional[torch.Tensor] = None
    requires_padding: bool = False


@dataclass
class IndexerMetadata:
    slot_mapping: torch.Tensor       # int64 [tokens]
    num_decodes: int = 0
    num_prefills: int = 0
    num_decode_tokens: int = 0
    prefill: Optional[PrefillMetadata] = None
    decode: Optional[DecodeMetadata] = None


def _cache_2d(kv_cache: torch.Tensor, head_dim: int):
    page_size = kv_cache.shape[1]
    c = kv_cache.reshape(kv_cache.shape[0], -1)
    if c.dtype != torch.uint8:
        c = c.view(torch.uint8)
    if c.shape[1] != page_size * (head_dim + 4):
        raise B200DSAError("kv_cache must hold page_size*(head_dim+4) bytes per block")
    return c.contiguous(), page_size


def _routed_rows(q_rows, w_rows, head_idx, cache, page_size, row_ctx, tables, row_table, next_n, cfg: M.MisaConfig,
                 n_keep: int, max_cols: int, use_misa: bool, req_lens):
    """Top-k positions (relative to the request start) for a set of query rows."""
    w_rows = w_rows.to(torch.float32).contiguous()
    kw = dict(next_n=next_n, max_cols=max_cols, row_table=row_table)
    if not use_misa:
        logits = K.indexer_paged_fp8_logits(q_rows, w_rows, cache, page_size, row_ctx, tables, **kw)
        return K.topk_select(logits, cfg.index_topk, col_end=row_ctx, sorted=True)
    if cfg.misa_use_qnorm:
        if head_idx is None:
            raise B200DSAError("misa_use_qnorm needs q_head_topk_indices")
        w_gate = M.gate_weights_by_heads(w_rows, head_idx[:, :n_keep])
    else:
        kb = cfg.misa_k_block_size
        max_pool = (max_cols + kb - 1) // kb
        pooled = K.paged_mean_pool_fp8(cache, page_size, req_lens, tables, kb, max_pool)
        n_pool = ((row_ctx + kb - 1) // kb).to(torch.int32).contiguous()
        rows = row_ctx.numel()
        req = row_table if row_table is not None else \
            (torch.arange(rows, device=row_ctx.device, dtype=torch.int32) // next_n).contiguous()
        w_gate, _ = K.router_block_score_topk(q_rows.to(torch.bfloat16), w_rows, pooled, torch.zeros_like(n_pool),
                                              n_pool, n_keep, pooled_set=req)
    s1 = min(cfg.misa_stage1_topk, max_cols)
    stage1 = K.indexer_paged_fp8_logits(q_rows, w_gate, cache, page_size, row_ctx, tables, **kw)
    cand = K.topk_select(stage1, s1, col_end=row_ctx, sorted=False)
    full = K.indexer_paged_fp8_logits(q_rows, w_rows, cache, page_size, row_ctx, tables, out=stage1, **kw)
    logits = torch.gather(full, 1, cand.clamp(min=0).long())
    logits = torch.where(cand >= 0, logits, torch.full_like(logits, float("-inf")))
    return M.misa_final_topk(logits, cand, cfg.index_topk)


@torch.no_grad()
def misa_sparse_attn_indexer(hidden_states: torch.Tensor, k_cache_prefix: str, kv_cache: torch.Tensor,
                             q_fp8: torch.Tensor, k: torch.Tensor, weights: torch.Tensor,
                             q_head_topk_indices: Optional[torch.Tensor], quant_block_size: int,
                             scale_fmt: Optional[str], topk_heads: int, decode_topk_heads: int, use_qnorm: bool,
                             k_block_size: Optional[int], stage1_topk: int, topk_tokens: int, head_dim: int,
                             max_model_len: int, total_seq_lens: int, topk_indices_buffer: torch.Tensor,
                             attn_metadata=None, use_misa: bool = True) -> torch.Tensor:
    """Same positional arguments as the reference op; `attn_metadata` (optional, last) replaces
    the forward-context lookup, `use_misa=False` gives the dense DSA baseline."""
    if attn_metadata is None:
        try:
            from vllm.forward_context import get_forward_context
            attn_metadata = get_forward_context().attn_metadata
        except Exception:  # noqa: BLE001
            attn_metadata = None
    if isinstance(attn_metadata, dict):
        attn_metadata = attn_metadata[k_cache_prefix]
    if attn_metadata is None or not hasattr(attn_metadata, "slot_mapping"):
        return topk_indices_buffer          # profiling / dummy run: leave the buffer untouched
    if head_dim != 128:
        raise B200DSAError("index head_dim must be 128")
    md = attn_metadata
    cache, page_size = _cache_2d(kv_cache, head_dim)
    cfg = M.MisaConfig(misa_topk_heads=topk_heads, misa_decode_topk_heads=decode_topk_heads,
                       misa_k_block_size=k_block_size or 1024, misa_use_qnorm=use_qnorm,
                       misa_stage1_topk=stage1_topk, index_topk=topk_tokens)
    n_tok = md.slot_mapping.shape[0]
    K.indexer_k_quant_and_cache(k[:n_tok].to(torch.bfloat16).contiguous(), cache, md.slot_mapping.contiguous(),
                                page_size)
    if cache.data_ptr() != kv_cache.data_ptr():
        raise B200DSAError("kv_cache must be contiguous so that it can be updated in place")
    topk_indices_buffer[: hidden_states.shape[0]] = -1
    kq = min(topk_tokens, topk_indices_buffer.shape[1])

    if md.num_prefills > 0 and md.prefill is not None:
        for ch in md.prefill.chunks:
            t0, t1 = ch.token_start, ch.token_end
            ks = ch.cu_seqlen_ks.to(torch.int32)
            ke = ch.cu_seqlen_ke.to(torch.int32)
            cu = ch.cu_seq_lens.to(torch.int32)
            req = (torch.searchsorted(cu, ks, right=True) - 1).to(torch.int32).contiguous()
            row_ctx = (ke - ks).clamp(min=0).contiguous()
            req_lens = (cu[1:] - cu[:-1]).contiguous()
            tables = ch.block_table.to(torch.int32).contiguous()
            max_cols = min(max_model_len, tables.shape[1] * page_size)
            hi = None if q_head_topk_indices is None else q_head_topk_indices[t0:t1]
            idx = _routed_rows(q_fp8[t0:t1].contiguous(), weights[t0:t1], hi, cache, page_size, row_ctx, tables,
                               req, 1, cfg, topk_heads, max_cols, use_misa, req_lens)
            topk_indices_buffer[t0:t1, :kq] = idx[:, :kq]

    if md.num_decodes > 0 and md.decode is not None:
        dm = md.decode
        nd = md.num_decode_tokens
        if dm.requires_padding:
            raise B200DSAError("padded decode batches (mixed decode lengths) are not supported")
        B = dm.seq_lens.shape[0]
        next_n = nd // B
        seq = dm.seq_lens.to(torch.int32)
        n_off = torch.arange(next_n, device=seq.device, dtype=torch.int32)
        row_ctx = (seq.view(-1, 1) - next_n + n_off.view(1, -1) + 1).clamp(min=0).reshape(-1).contiguous()
        tables = dm.block_table.to(torch.int32).contiguous()
        max_cols = min(max_model_len, tables.shape[1] * page_size)
        hi = None if q_head_topk_indices is None else q_head_topk_indices[:nd]
        idx = _routed_rows(q_fp8[:nd].contiguous(), weights[:nd], hi, cache, page_size, row_ctx, tables, None,
                           next_n, cfg, decode_topk_heads, max_cols, use_misa, seq.contiguous())
        topk_indices_buffer[:nd, :kq] = idx[:, :kq]
    return topk_indices_buffer


class MiSASparseAttnIndexer(torch.nn.Module):
    """Constructor and forward signatures of the reference's CustomOp (indexers.py:628-712)."""

    use_misa = True

    def __init__(self, k_cache, quant_block_size: int, scale_fmt: Optional[str], topk_heads: int,
                 decode_topk_heads: int, use_qnorm: bool, k_block_size: Optional[int], stage1_topk: int,
                 topk_tokens: int, head_dim: int, max_model_len: int, max_total_seq_len: int,
                 topk_indices_buffer: torch.Tensor):
        super().__init__()
        self.k_cache = k_cache
        self.quant_block_size, self.scale_fmt = quant_block_size, scale_fmt
        self.topk_heads, self.decode_topk_heads = topk_heads, decode_topk_heads
        self.use_qnorm, self.k_block_size, self.stage1_topk = use_qnorm, k_block_size, stage1_topk
        self.topk_tokens, self.head_dim = topk_tokens, head_dim
        self.max_model_len, self.max_total_seq_len = max_model_len, max_total_seq_len
        self.topk_indices_buffer = topk_indices_buffer

    def _cache_tensor(self):
        kc = self.k_cache
        if isinstance(kc, torch.Tensor):
            return kc, ""
        return kc.kv_cache[0], getattr(kc, "prefix", "")     # vLLM's cache holder object

    def forward_cuda(self, hidden_states, q_fp8, k, weights, q_head_topk_indices=None, attn_metadata=None):
        cache, prefix = self._cache_tensor()
        return misa_sparse_attn_indexer(hidden_states, prefix, cache, q_fp8, k, weights, q_head_topk_indices,
                                        self.quant_block_size, self.scale_fmt, self.topk_heads,
                                        self.decode_topk_heads, self.use_qnorm, self.k_block_size, self.stage1_topk,
                                        self.topk_tokens, self.head_dim, self.max_model_len, self.max_total_seq_len,
                                        self.topk_indices_buffer, attn_metadata=attn_metadata,
                                        use_misa=self.use_misa)

    forward = forward_cuda

    def forward_native(self, *args, **kwargs):
        raise B200DSAError("there is no native (non-CUDA) path for the indexer")


class BaselineSparseAttnIndexer(MiSASparseAttnIndexer):
    """Dense DSA indexer (all 64 heads, no stage-1 shortlist): forward_cuda(hidden_states, q_fp8, k, weights)."""

    use_misa = False

    def __init__(self, k_cache, quant_block_size, scale_fmt, topk_tokens, head_dim, max_model_len,
                 max_total_seq_len, topk_indices_buffer):
        super().__init__(k_cache, quant_block_size, scale_fmt, 64, 64, True, None, topk_tokens, topk_tokens,
                         head_dim, max_model_len, max_total_seq_len, topk_indices_buffer)


def register() -> None:
    """Register the hook as a torch custom op named like the reference's
    (indexers.py:607-613: mutates topk_indices_buffer, with a fake implementation for tracing).
    Calling it again is a no-op."""
    if getattr(register, "_lib", None) is not None:
        return
    lib = torch.library.Library("b200dsa", "FRAGMENT")
    lib.define("misa_sparse_attn_indexer(Tensor hidden_states, str k_cache_prefix, Tensor kv_cache, Tensor q_fp8, "
               "Tensor k, Tensor weights, Tensor? q_head_topk_indices, int quant_block_size, str? scale_fmt, "
               "int topk_heads, int decode_topk_heads, bool use_qnorm, int? k_block_size, int stage1_topk, "
               "int topk_tokens, int head_dim, int max_model_len, int total_seq_lens, "
               "Tensor(a!) topk_indices_buffer) -> Tensor")
    lib.impl("misa_sparse_attn_indexer", misa_sparse_attn_indexer, "CUDA")
    lib.impl("misa_sparse_attn_indexer", lambda *a, **k: a[-1], "Meta")
    register._lib = lib  # keep alive
