"""Indexer-backend hook with the reference's vLLM signatures.

    MiSASparseAttnIndexer.forward_cuda(hidden_states, q_fp8, k, weights, q_head_topk_indices)
        MISA_preprint/misa_vllm_patch_2stage/misa_vllm_patch/indexers.py:628-712
    misa_sparse_attn_indexer(...)        same file :388-581 (the custom op it wraps)
    BaselineSparseAttnIndexer            same file :333-354 (dense DSA twin, no head routing)
    baseline_sparse_attn_indexer(...)    same file :36-232
    register()                           misa_vllm_patch/register.py:1-8, found by vLLM through the
                                         "vllm.general_plugins" entry point of pyproject.toml:4-5

When vLLM is importable the two classes ARE vllm CustomOp subclasses registered under the
reference's names, and the two functions are registered as torch.ops.vllm.* with
mutates_args=["topk_indices_buffer"] and a fake implementation, exactly as the reference does at
indexers.py:607-613; without vLLM they are plain torch modules and the ops live at
torch.ops.b200dsa.*.  `SparseAttnIndexer022` adapts the constructor and forward_cuda signature of the
vLLM 0.22 layer (vllm/model_executor/layers/sparse_attn_indexer.py), whose decode metadata may carry
per-row context lengths [B, next_n] and has no use_large_context_topk / offsets fields.

What the op does per step: insert the new index keys into the paged FP8 cache, fill
topk_indices_buffer with -1, then for prefill chunks and for decode rows score the cached keys
and write each token's top-k key positions *relative to its request's first key* (int32, -1
padded) into its row of the buffer.  The buffer object itself is always returned (the
reference returns None on prefill-only steps, indexers.py:581).

Metadata: vLLM hands the op a per-layer metadata object through its forward context.  The
fields read here are the ones the reference reads (indexers.py:443-446, :474-495, :521-565);
any object with these attributes works, and the small dataclasses below can be filled
directly by tests.  When `attn_metadata` is not passed and vLLM is importable, it is taken from
vllm.forward_context as the reference does.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

import torch

from . import kernels as K
from . import misa as M
from ._lib import B200DSAError

try:  # the reference's base class, when the serving engine is installed
    from vllm.model_executor.custom_op import CustomOp as _OpBase
    HAVE_VLLM = True
except Exception:  # noqa: BLE001 - any import problem means "no vLLM here"
    _OpBase = torch.nn.Module
    HAVE_VLLM = False


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
    seq_lens: torch.Tensor           # int32 [B], or [B, next_n] per-row contexts (vLLM 0.22 MTP path)
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
    """Top-k positions (relative to the request start) for a set of query rows.  The cache is read
    ONCE: with head routing the indexer kernel writes the routed stage-1 score and the all-head
    score of every key in the same pass (head bit mask), and stage 2 is a gather."""
    w_rows = w_rows.to(torch.float32).contiguous()
    kw = dict(next_n=next_n, max_cols=max_cols, row_table=row_table, fill=False)
    if not use_misa:
        logits = K.indexer_paged_fp8_logits(q_rows, w_rows, cache, page_size, row_ctx, tables, **kw)
        return K.topk_select(logits, min(cfg.index_topk, max_cols), col_end=row_ctx, sorted=True)
    if cfg.misa_use_qnorm:
        if head_idx is None:
            raise B200DSAError("misa_use_qnorm needs q_head_topk_indices")
        head_idx = head_idx[:, :n_keep]
    else:
        kb = cfg.misa_k_block_size
        max_pool = (max_cols + kb - 1) // kb
        pooled = K.paged_mean_pool_fp8(cache, page_size, req_lens, tables, kb, max_pool)
        n_pool = ((row_ctx + kb - 1) // kb).to(torch.int32).contiguous()
        rows = row_ctx.numel()
        req = row_table if row_table is not None else \
            (torch.arange(rows, device=row_ctx.device, dtype=torch.int32) // next_n).contiguous()
        _, head_idx = K.router_block_score_topk(q_rows.to(torch.bfloat16), w_rows, pooled, torch.zeros_like(n_pool),
                                                n_pool, n_keep, pooled_set=req)
    s1 = min(cfg.misa_stage1_topk, max_cols)
    full, stage1 = K.indexer_paged_fp8_logits(q_rows, w_rows, cache, page_size, row_ctx, tables,
                                              head_mask=K.head_mask_from_indices(head_idx), **kw)
    cand = K.topk_select(stage1, s1, col_end=row_ctx, sorted=False)
    logits = torch.gather(full, 1, cand.clamp(min=0).long())
    logits = torch.where(cand >= 0, logits, torch.full_like(logits, float("-inf")))
    return M.misa_final_topk(logits, cand, cfg.index_topk)


def _decode_rows(dm, nd: int):
    """Per decode token: (row_ctx int32 [nd] keys visible, row_table int32 [nd] or None, next_n).

    Uniform batches: token (b, j) sees seq_len[b] - next_n + j + 1 keys (indexers.py:545-551).
    vLLM 0.22 may hand these contexts over directly as seq_lens [B, next_n].  Padded batches
    (requires_padding, requests with different decode lengths, indexers.py:165-171 / :237-240):
    the reference pads every request to next_n = max(decode_lens) rows, scores the padded layout
    and unpacks; the same numbers come out of scoring only the real tokens with next_n taken as
    that maximum, so nothing is padded here.  That branch reads max(decode_lens) on the host."""
    seq = dm.seq_lens.to(torch.int32)
    B = seq.shape[0]
    if seq.dim() == 2:
        return seq.reshape(-1)[:nd].contiguous(), None, seq.shape[1]
    if not getattr(dm, "requires_padding", False):
        next_n = max(1, nd // max(B, 1))
        n_off = torch.arange(next_n, device=seq.device, dtype=torch.int32)
        row_ctx = (seq.view(-1, 1) - next_n + n_off.view(1, -1) + 1).clamp(min=0).reshape(-1)
        return row_ctx.contiguous(), None, next_n
    dl = dm.decode_lens.to(torch.int64)
    next_n = int(dl.max())
    req = torch.repeat_interleave(torch.arange(B, device=seq.device), dl, output_size=nd)
    first = torch.cumsum(dl, 0) - dl
    j = torch.arange(nd, device=seq.device) - first[req]
    row_ctx = (seq[req].long() - next_n + j + 1).clamp(min=0).to(torch.int32)
    return row_ctx.contiguous(), req.to(torch.int32).contiguous(), 1


@torch.no_grad()
def misa_sparse_attn_indexer(hidden_states: torch.Tensor, k_cache_prefix: str, kv_cache: torch.Tensor,
                             q_fp8: torch.Tensor, k: torch.Tensor, weights: torch.Tensor,
                             q_head_topk_indices: Optional[torch.Tensor], quant_block_size: int,
                             scale_fmt: Optional[str], topk_heads: int, decode_topk_heads: int, use_qnorm: bool,
                             k_block_size: Optional[int], stage1_topk: int, topk_tokens: int, head_dim: int,
                             max_model_len: int, total_seq_lens: int, topk_indices_buffer: torch.Tensor,
                             attn_metadata=None, use_misa: bool = True, skip_k_cache_insert: bool = False
                             ) -> torch.Tensor:
    """Same positional arguments as the reference op; `attn_metadata` (optional) replaces
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
    if head_dim != 128 or quant_block_size != 128:
        raise B200DSAError("index head_dim and quant_block_size must be 128")
    if scale_fmt not in (None, "ue8m0"):
        raise B200DSAError(f"unknown scale_fmt {scale_fmt!r} (None or 'ue8m0')")
    md = attn_metadata
    cache, page_size = _cache_2d(kv_cache, head_dim)
    if cache.data_ptr() != kv_cache.data_ptr():
        raise B200DSAError("kv_cache must be contiguous so that it can be updated in place")
    cfg = M.MisaConfig(misa_topk_heads=topk_heads, misa_decode_topk_heads=decode_topk_heads,
                       misa_k_block_size=k_block_size or 1024, misa_use_qnorm=use_qnorm,
                       misa_stage1_topk=stage1_topk, index_topk=topk_tokens)
    n_tok = md.slot_mapping.shape[0]
    if not skip_k_cache_insert:
        K.indexer_k_quant_and_cache(k[:n_tok].to(torch.bfloat16).contiguous(), cache, md.slot_mapping.contiguous(),
                                    page_size, scale_fmt)
    topk_indices_buffer[: hidden_states.shape[0]] = -1
    kq = min(topk_tokens, topk_indices_buffer.shape[1])

    if md.num_prefills > 0 and md.prefill is not None:
        for ch in md.prefill.chunks:
            t0, t1 = ch.token_start, ch.token_end
            ks = ch.cu_seqlen_ks.to(torch.int32)
            ke = ch.cu_seqlen_ke.to(torch.int32)
            cu = ch.cu_seq_lens.to(torch.int32)
            tok2seq = getattr(ch, "token_to_seq", None)
            req = (tok2seq if tok2seq is not None else torch.searchsorted(cu, ks, right=True) - 1)
            req = req.to(torch.int32).contiguous()
            row_ctx = (ke - ks).clamp(min=0).contiguous()
            req_lens = (cu[1:] - cu[:-1]).contiguous()
            tables = ch.block_table.to(torch.int32).contiguous()
            max_cols = min(max_model_len, tables.shape[1] * page_size)
            hi = None if q_head_topk_indices is None else q_head_topk_indices[t0:t1]
            idx = _routed_rows(q_fp8[t0:t1].contiguous(), weights[t0:t1], hi, cache, page_size, row_ctx, tables,
                               req, 1, cfg, topk_heads, max_cols, use_misa, req_lens)
            n = min(kq, idx.shape[1])      # fewer columns when stage1_topk or the block table is short
            topk_indices_buffer[t0:t1, :n] = idx[:, :n]

    if md.num_decodes > 0 and md.decode is not None:
        dm = md.decode
        nd = md.num_decode_tokens
        row_ctx, row_table, next_n = _decode_rows(dm, nd)
        seq = dm.seq_lens.to(torch.int32)
        req_lens = (seq if seq.dim() == 1 else seq.max(dim=1).values).contiguous()
        tables = dm.block_table.to(torch.int32).contiguous()
        max_cols = min(max_model_len, tables.shape[1] * page_size)
        hi = None if q_head_topk_indices is None else q_head_topk_indices[:nd]
        idx = _routed_rows(q_fp8[:nd].contiguous(), weights[:nd], hi, cache, page_size, row_ctx, tables, row_table,
                           next_n, cfg, decode_topk_heads, max_cols, use_misa, req_lens)
        n = min(kq, idx.shape[1])
        topk_indices_buffer[:nd, :n] = idx[:, :n]
    return topk_indices_buffer


# ------------------------------------------------------------------------------------------
# The two ops under the reference's exact schemas (19 and 12 arguments, indexers.py:388-408, :36-49)
# ------------------------------------------------------------------------------------------
def _misa_op(hidden_states: torch.Tensor, k_cache_prefix: str, kv_cache: torch.Tensor, q_fp8: torch.Tensor,
             k: torch.Tensor, weights: torch.Tensor, q_head_topk_indices: Optional[torch.Tensor],
             quant_block_size: int, scale_fmt: Optional[str], topk_heads: int, decode_topk_heads: int,
             use_qnorm: bool, k_block_size: Optional[int], stage1_topk: int, topk_tokens: int, head_dim: int,
             max_model_len: int, total_seq_lens: int, topk_indices_buffer: torch.Tensor) -> torch.Tensor:
    return misa_sparse_attn_indexer(hidden_states, k_cache_prefix, kv_cache, q_fp8, k, weights, q_head_topk_indices,
                                    quant_block_size, scale_fmt, topk_heads, decode_topk_heads, use_qnorm,
                                    k_block_size, stage1_topk, topk_tokens, head_dim, max_model_len, total_seq_lens,
                                    topk_indices_buffer)


def _misa_op_fake(hidden_states: torch.Tensor, k_cache_prefix: str, kv_cache: torch.Tensor, q_fp8: torch.Tensor,
                  k: torch.Tensor, weights: torch.Tensor, q_head_topk_indices: Optional[torch.Tensor],
                  quant_block_size: int, scale_fmt: Optional[str], topk_heads: int, decode_topk_heads: int,
                  use_qnorm: bool, k_block_size: Optional[int], stage1_topk: int, topk_tokens: int, head_dim: int,
                  max_model_len: int, total_seq_lens: int, topk_indices_buffer: torch.Tensor) -> torch.Tensor:
    return topk_indices_buffer


def baseline_sparse_attn_indexer(hidden_states: torch.Tensor, k_cache_prefix: str, kv_cache: torch.Tensor,
                                 q_fp8: torch.Tensor, k: torch.Tensor, weights: torch.Tensor, quant_block_size: int,
                                 scale_fmt: Optional[str], topk_tokens: int, head_dim: int, max_model_len: int,
                                 total_seq_lens: int, topk_indices_buffer: torch.Tensor) -> torch.Tensor:
    """Dense DSA indexer op, arguments of indexers.py:36-49."""
    return misa_sparse_attn_indexer(hidden_states, k_cache_prefix, kv_cache, q_fp8, k, weights, None,
                                    quant_block_size, scale_fmt, 64, 64, True, None, topk_tokens, topk_tokens,
                                    head_dim, max_model_len, total_seq_lens, topk_indices_buffer, use_misa=False)


def _baseline_op_fake(hidden_states: torch.Tensor, k_cache_prefix: str, kv_cache: torch.Tensor,
                      q_fp8: torch.Tensor, k: torch.Tensor, weights: torch.Tensor, quant_block_size: int,
                      scale_fmt: Optional[str], topk_tokens: int, head_dim: int, max_model_len: int,
                      total_seq_lens: int, topk_indices_buffer: torch.Tensor) -> torch.Tensor:
    return topk_indices_buffer


OP_NAMESPACE = "vllm" if HAVE_VLLM else "b200dsa"
MISA_OP_NAME = "misa_sparse_attn_indexer"
BASELINE_OP_NAME = "baseline_sparse_attn_indexer"
_own_lib = None


def register_ops() -> str:
    """Register both ops (idempotent).  With vLLM: torch.ops.vllm.<name> through vLLM's own
    direct_register_custom_op, CUDA dispatch key, mutates_args=["topk_indices_buffer"], fake
    implementation returning the buffer (indexers.py:607-613, :271-277).  Without vLLM: the same
    schemas under torch.ops.b200dsa.  Returns the namespace used."""
    global _own_lib
    ns = getattr(torch.ops, OP_NAMESPACE)
    if hasattr(ns, MISA_OP_NAME) and hasattr(ns, BASELINE_OP_NAME):
        return OP_NAMESPACE
    if HAVE_VLLM:
        from vllm.utils.torch_utils import direct_register_custom_op
        for name, fn, fake in ((MISA_OP_NAME, _misa_op, _misa_op_fake),
                               (BASELINE_OP_NAME, baseline_sparse_attn_indexer, _baseline_op_fake)):
            if not hasattr(ns, name):
                direct_register_custom_op(op_name=name, op_func=fn, mutates_args=["topk_indices_buffer"],
                                          fake_impl=fake, dispatch_key="CUDA")
        return OP_NAMESPACE
    _own_lib = torch.library.Library(OP_NAMESPACE, "FRAGMENT")
    for name, fn, fake in ((MISA_OP_NAME, _misa_op, _misa_op_fake),
                           (BASELINE_OP_NAME, baseline_sparse_attn_indexer, _baseline_op_fake)):
        schema = torch.library.infer_schema(fn, mutates_args=["topk_indices_buffer"])
        _own_lib.define(name + schema)
        _own_lib.impl(name, fn, "CUDA")
        _own_lib._register_fake(name, fake)
    return OP_NAMESPACE


def _cache_and_prefix(k_cache):
    if isinstance(k_cache, torch.Tensor):
        return k_cache, ""
    kc = k_cache.kv_cache
    if isinstance(kc, (list, tuple)):      # vLLM 0.17 keeps one tensor per virtual engine
        kc = kc[0]
    return kc, getattr(k_cache, "prefix", "")


def _op_base_init(self):
    if HAVE_VLLM:
        try:
            _OpBase.__init__(self)
            return
        except Exception:  # noqa: BLE001 - no vLLM config in scope (tests, stand-alone use): plain module
            pass
    torch.nn.Module.__init__(self)


class MiSASparseAttnIndexer(_OpBase):
    """Constructor and forward signatures of the reference's CustomOp (indexers.py:628-712)."""

    use_misa = True

    def __init__(self, k_cache, quant_block_size: int, scale_fmt: Optional[str], topk_heads: int,
                 decode_topk_heads: int, use_qnorm: bool, k_block_size: Optional[int], stage1_topk: int,
                 topk_tokens: int, head_dim: int, max_model_len: int, max_total_seq_len: int,
                 topk_indices_buffer: torch.Tensor):
        _op_base_init(self)
        self.k_cache = k_cache
        self.quant_block_size, self.scale_fmt = quant_block_size, scale_fmt
        self.topk_heads, self.decode_topk_heads = topk_heads, decode_topk_heads
        self.use_qnorm, self.k_block_size, self.stage1_topk = use_qnorm, k_block_size, stage1_topk
        self.topk_tokens, self.head_dim = topk_tokens, head_dim
        self.max_model_len, self.max_total_seq_len = max_model_len, max_total_seq_len
        self.topk_indices_buffer = topk_indices_buffer

    def forward_cuda(self, hidden_states, q_fp8, k, weights, q_head_topk_indices=None, attn_metadata=None):
        cache, prefix = _cache_and_prefix(self.k_cache)
        if attn_metadata is None and not isinstance(self.k_cache, torch.Tensor):
            # inside the engine: through the registered op, as the reference does (indexers.py:684-712)
            op = getattr(getattr(torch.ops, register_ops()), MISA_OP_NAME if self.use_misa else BASELINE_OP_NAME)
            if self.use_misa:
                return op(hidden_states, prefix, cache, q_fp8, k, weights, q_head_topk_indices,
                          self.quant_block_size, self.scale_fmt, self.topk_heads, self.decode_topk_heads,
                          self.use_qnorm, self.k_block_size, self.stage1_topk, self.topk_tokens, self.head_dim,
                          self.max_model_len, self.max_total_seq_len, self.topk_indices_buffer)
            return op(hidden_states, prefix, cache, q_fp8, k, weights, self.quant_block_size, self.scale_fmt,
                      self.topk_tokens, self.head_dim, self.max_model_len, self.max_total_seq_len,
                      self.topk_indices_buffer)
        return misa_sparse_attn_indexer(hidden_states, prefix, cache, q_fp8, k, weights, q_head_topk_indices,
                                        self.quant_block_size, self.scale_fmt, self.topk_heads,
                                        self.decode_topk_heads, self.use_qnorm, self.k_block_size, self.stage1_topk,
                                        self.topk_tokens, self.head_dim, self.max_model_len, self.max_total_seq_len,
                                        self.topk_indices_buffer, attn_metadata=attn_metadata,
                                        use_misa=self.use_misa)

    def forward(self, *args, **kwargs):
        return self.forward_cuda(*args, **kwargs)

    def forward_native(self, *args, **kwargs):
        # the reference routes the "native" path to the CUDA one as well (indexers.py:659-682)
        return self.forward_cuda(*args, **kwargs)


class BaselineSparseAttnIndexer(MiSASparseAttnIndexer):
    """Dense DSA indexer (all 64 heads, no stage-1 shortlist): forward_cuda(hidden_states, q_fp8, k, weights)
    (indexers.py:279-386)."""

    use_misa = False

    def __init__(self, k_cache, quant_block_size, scale_fmt, topk_tokens, head_dim, max_model_len,
                 max_total_seq_len, topk_indices_buffer):
        super().__init__(k_cache, quant_block_size, scale_fmt, 64, 64, True, None, topk_tokens, topk_tokens,
                         head_dim, max_model_len, max_total_seq_len, topk_indices_buffer)


class SparseAttnIndexer022(BaselineSparseAttnIndexer):
    """The dense indexer behind the constructor and forward_cuda(hidden_states, q_quant, k, weights) of
    vLLM 0.22's SparseAttnIndexer layer.  q_quant must be the FP8 tensor (per-token scale folded into
    `weights`); the FP4 cache variant of that layer is not supported."""

    def __init__(self, k_cache, quant_block_size: int, scale_fmt: Optional[str], topk_tokens: int, head_dim: int,
                 max_model_len: int, max_total_seq_len: int, topk_indices_buffer: torch.Tensor,
                 skip_k_cache_insert: bool = False, use_fp4_cache: bool = False):
        if use_fp4_cache:
            raise B200DSAError("the FP4 index-key cache is not supported")
        super().__init__(k_cache, quant_block_size, scale_fmt, topk_tokens, head_dim, max_model_len,
                         max_total_seq_len, topk_indices_buffer)
        self.skip_k_cache_insert = skip_k_cache_insert

    def forward_cuda(self, hidden_states, q_quant, k, weights, attn_metadata=None):
        if isinstance(q_quant, tuple):
            raise B200DSAError("q_quant must be a single FP8 tensor (the FP4 path passes a tuple)")
        cache, prefix = _cache_and_prefix(self.k_cache)
        return misa_sparse_attn_indexer(hidden_states, prefix, cache, q_quant, k, weights, None,
                                        self.quant_block_size, self.scale_fmt, 64, 64, True, None,
                                        self.topk_tokens, self.topk_tokens, self.head_dim, self.max_model_len,
                                        self.max_total_seq_len, self.topk_indices_buffer,
                                        attn_metadata=attn_metadata, use_misa=False,
                                        skip_k_cache_insert=self.skip_k_cache_insert)


def _register_custom_op_classes() -> None:
    """Enter the classes into vLLM's CustomOp registry under the reference's names
    (indexers.py:279 "baseline_sparse_attn_indexer", :615 "misa_sparse_attn_indexer")."""
    if not HAVE_VLLM:
        return
    from vllm.model_executor import custom_op as co
    for name, cls in ((MISA_OP_NAME, MiSASparseAttnIndexer), (BASELINE_OP_NAME, BaselineSparseAttnIndexer),
                      ("b200dsa_sparse_attn_indexer", SparseAttnIndexer022)):
        if name not in co.op_registry:
            _OpBase.register(name)(cls)


def register() -> None:
    """Plugin entry point ("vllm.general_plugins"): registers the two torch ops and the CustomOp
    classes.  Calling it again is a no-op.  The reference's register() additionally enters its
    model class MiSAForCausalLM into vLLM's ModelRegistry (register.py:2-8); the model definition
    is outside this library, which provides the indexer op that model constructs."""
    register_ops()
    _register_custom_op_classes()
