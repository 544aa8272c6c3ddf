"""Drop-in replacements for OpenDSA's selection ops, same names and argument meaning:

    indexer_select_topk            OpenDSA/opendsa/ops/topk_select.py:30-72
    sparse_attend_absorbed_chunked OpenDSA/opendsa/ops/sparse_mla.py:51-103
    prepare_ks_ke / prepare_ks_ke_cp  OpenDSA/opendsa/ops/flashkl_warmup.py:41-56, :235-248

The selection is forward-only (the reference's is under torch.no_grad).  The sparse attention is
differentiable in q_lat, latent and W_UV: its forward is the attention and up-projection kernels, its
backward rebuilds the probabilities from the saved log-sum-exp per query chunk and runs as library
GEMMs.  Tensors must live on a CUDA device; there is no CPU path.  `patch_opendsa()` rebinds the names the reference imported at module load
(OpenDSA/opendsa/modeling/dsa_attention.py:31-38).

Numerics: scores are computed from bf16-rounded q and k with fp32 accumulation on tcgen05
tensor cores (the reference computes in the dtype it is given); attention runs in bf16 with
fp32 softmax and accumulation.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import kernels as K
from ._lib import B200DSAError

_BLOCK = 128
_MAX_LOGIT_BYTES = 1 << 30   # scratch bound for one query chunk of token logits


def prepare_ks_ke(cu_seqlens: torch.Tensor, total: Optional[int] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per packed query the causal interval [ks, ke): ks = start of its document,
    ke = its own position + 1.  Device-side; `total` (the number of packed tokens, cu_seqlens[-1])
    saves the one host synchronisation that reading it costs."""
    cu = cu_seqlens.to(torch.int64)
    if total is None:
        total = int(cu[-1]) if cu.numel() else 0
    t = torch.arange(total, dtype=torch.int64, device=cu.device)
    doc = torch.searchsorted(cu, t, right=True) - 1
    return cu[doc], t + 1


def prepare_ks_ke_cp(cu_full: torch.Tensor, q_global_pos: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Intervals for local queries that sit at global positions (context parallel / decode)."""
    cu = cu_full.to(torch.int64)
    p = q_global_pos.to(torch.int64)
    d = (torch.searchsorted(cu, p, right=True) - 1).clamp(0, cu.numel() - 2)
    return cu[d], p + 1


def _pad_heads(q: torch.Tensor, w: torch.Tensor):
    """The kernels score exactly 64 index heads; fewer heads are padded with zero weight."""
    H = q.shape[1]
    if H == 64:
        return q.contiguous(), w.contiguous()
    if H > 64:
        raise B200DSAError("at most 64 index heads are supported")
    qp = q.new_zeros(q.shape[0], 64, q.shape[2])
    qp[:, :H] = q
    wp = w.new_zeros(w.shape[0], 64)
    wp[:, :H] = w
    return qp, wp


def identity_block_lists(ks: torch.Tensor, ke: torch.Tensor, n_keys: int):
    """Per row the list of 128-key blocks covering [ks, ke): (block_list int32 [T, max_blocks]
    padded with -1, row_cols int32 [T])."""
    nb_total = (n_keys + _BLOCK - 1) // _BLOCK
    b0 = (ks // _BLOCK).to(torch.int32)
    b1 = ((ke + _BLOCK - 1) // _BLOCK).to(torch.int32)
    nblk = (b1 - b0).clamp(min=0)
    j = torch.arange(nb_total, dtype=torch.int32, device=ks.device).view(1, -1)
    bl = torch.where(j < nblk.view(-1, 1), b0.view(-1, 1) + j, torch.full_like(j, -1))
    return bl.contiguous(), (nblk * _BLOCK).to(torch.int32)


def indexer_logits_flat(q: torch.Tensor, k: torch.Tensor, w: torch.Tensor, ks: torch.Tensor, ke: torch.Tensor,
                        sm_scale: float, out: Optional[torch.Tensor] = None):
    """Token logits of every row over the 128-key blocks covering its interval [ks, ke):
    (logits fp32 [T, cols] with -inf outside the interval, col0 int32 [T] = position of column 0 of
    each row, row_cols int32 [T]).  No block list is built: the kernel walks consecutive blocks, and four
    consecutive queries share every key tile.  With `out` (fp32 [>= T, >= cols]) nothing is allocated or
    pre-filled: only the columns below row_cols of each row are then defined."""
    lo = ks.to(torch.int32).contiguous()
    hi = ke.to(torch.int32).contiguous()
    col0 = (lo >> 7) << 7
    row_cols = (((hi + (_BLOCK - 1)) >> 7) << 7) - col0
    row_cols.clamp_(min=0)
    cols = ((k.shape[0] + _BLOCK - 1) // _BLOCK) * _BLOCK
    logits = K.indexer_flat_bf16_logits(q, w, k, lo, hi, row_cols.contiguous(), cols, out_scale=sm_scale, out=out)
    return logits[:q.shape[0]], col0, row_cols


@torch.no_grad()
def indexer_select_topk(index_q, index_k, index_w, cu_seqlens, topk, *, sm_scale_index: Optional[float] = None,
                        q_chunk: int = 4096, q_global_pos=None, sorted: bool = True) -> torch.Tensor:
    """Per-query top-k causal key positions by the lightning-indexer score
    I[t,j] = sm_scale * sum_h w[t,h] * relu(<q[t,h], k[j]>); int32 [Lq, topk], absolute
    positions in descending score order, -1 where fewer than topk keys are visible.
    sorted=False (not a reference argument) returns the same set of positions in no particular order:
    the attention that consumes them is order-invariant (OpenDSA/opendsa/ops/sparse_mla.py:39-43), and
    ordering 2048 winners per query costs more than scoring them."""
    if not index_q.is_cuda:
        raise B200DSAError("indexer_select_topk needs CUDA tensors (no CPU path)")
    Lq, H, d = index_q.shape
    if d != 128:
        raise B200DSAError("index head dim must be 128")
    sf = sm_scale_index if sm_scale_index is not None else d ** -0.5
    q, w = _pad_heads(index_q.to(torch.bfloat16), index_w.to(torch.float32))
    k = index_k.to(torch.bfloat16).contiguous()
    Lk = k.shape[0]
    if topk > 8192:
        raise B200DSAError("topk above 8192 is not supported")
    if Lq == 0 or Lk == 0:
        return torch.full((Lq, topk), -1, dtype=torch.int32, device=index_q.device)
    out = torch.empty(Lq, topk, dtype=torch.int32, device=index_q.device)     # the selection writes every column
    cols = ((Lk + _BLOCK - 1) // _BLOCK) * _BLOCK
    rows_per = max(1, min(q_chunk, _MAX_LOGIT_BYTES // (cols * 4)))
    k_eff = topk
    buf = torch.empty(min(rows_per, Lq), cols, dtype=torch.float32, device=index_q.device)   # read below row_cols only
    # the causal intervals of all queries and the column frame of their logits rows: one launch
    lo, hi, col0, row_cols = K.causal_row_intervals(cu_seqlens, Lq, q_global_pos)
    for t0 in range(0, Lq, rows_per):
        t1 = min(t0 + rows_per, Lq)
        logits = K.indexer_flat_bf16_logits(q[t0:t1], w[t0:t1], k, lo[t0:t1], hi[t0:t1], row_cols[t0:t1], cols,
                                            out_scale=sf, out=buf)
        K.topk_select(logits[:t1 - t0], k_eff, col_end=row_cols[t0:t1], row_pos_offset=col0[t0:t1], sorted=sorted,
                      out=out[t0:t1])
    return out


@torch.no_grad()
def sparse_attend_latent(q_lat, latent, indices, *, sm_scale: float, q_pos: Optional[torch.Tensor] = None,
                         ctx_dtype: torch.dtype = torch.float32):
    """Latent-space context and log-sum-exp: (ctx [L,H,512] fp32 or bf16, lse fp32 [L,H])."""
    if q_lat.shape[-1] != 576 or latent.shape[-1] != 576:
        raise B200DSAError("latent width must be 576 (512 value dims + 64 rope dims)")
    ctx = None
    if ctx_dtype == torch.bfloat16:
        ctx = torch.empty(q_lat.shape[0], q_lat.shape[1], 512, dtype=torch.bfloat16, device=q_lat.device)
    return K.sparse_mla_decode(q_lat.to(torch.bfloat16).contiguous(), latent.to(torch.bfloat16).contiguous(),
                               indices.to(torch.int32).contiguous(), sm_scale,
                               q_pos=None if q_pos is None else q_pos.to(torch.int32).contiguous(), ctx=ctx)


def _up_project(ctx: torch.Tensor, W_UV: torch.Tensor) -> torch.Tensor:
    """[L,H,512] latent context -> [L,H,Dv] through the per-head W_UV (tcgen05 kernel up to Dv = 256)."""
    if W_UV.shape[1] > 256:
        return torch.einsum("thl,hvl->thv", ctx.to(W_UV.dtype), W_UV)
    out_dtype = W_UV.dtype if W_UV.dtype in (torch.bfloat16, torch.float32) else torch.float32
    out = K.wuv_up_project(ctx, W_UV.to(torch.bfloat16).contiguous(), out_dtype=out_dtype)
    return out.to(W_UV.dtype)


class _SparseAttendAbsorbed(torch.autograd.Function):
    """Training form of the op.  Forward: the attention kernel (bf16 latent context + fp32 log-sum-exp)
    and the W_UV kernel; only (q, latent, W_UV, indices, q_pos, ctx, lse) are kept.  Backward: per chunk
    of queries the probabilities are rebuilt from the saved log-sum-exp (p = exp(s - lse), no second
    softmax pass: b200dsa_sparse_attn_bwd_pointwise), the five products of the attention backward run as
    library GEMMs on the gathered rows, and d_latent is accumulated in fp32 by
    b200dsa_scatter_add_latent_rows.  The reference reaches the same gradients by
    checkpointing _attend_absorbed_chunk and letting autograd replay it
    (OpenDSA/opendsa/ops/sparse_mla.py:26-48, :96-104)."""

    @staticmethod
    def forward(fctx, q_lat, latent, W_UV, indices, q_pos, sm_scale, q_chunk):
        ctx, lse = sparse_attend_latent(q_lat, latent, indices, sm_scale=sm_scale, q_pos=q_pos,
                                        ctx_dtype=torch.bfloat16)
        fctx.save_for_backward(q_lat, latent, W_UV, indices, q_pos, ctx, lse)
        fctx.sm_scale, fctx.q_chunk = sm_scale, q_chunk
        return _up_project(ctx, W_UV.detach())

    @staticmethod
    def backward(fctx, d_out):
        q_lat, latent, W_UV, indices, q_pos, ctx, lse = fctx.saved_tensors
        scale, L = fctx.sm_scale, q_lat.shape[0]
        # the five products run in the dtype of the inputs (bf16 inputs: bf16 operands on the tensor cores, fp32
        # accumulation, as the reference's own backward under bf16); the softmax algebra stays fp32
        cdt = torch.bfloat16 if q_lat.dtype == torch.bfloat16 and latent.dtype == torch.bfloat16 else torch.float32
        lat = latent.detach().to(cdt)
        Wc = W_UV.detach().to(cdt)
        need_q, need_l, need_w = fctx.needs_input_grad[0], fctx.needs_input_grad[1], fctx.needs_input_grad[2]
        d_q = torch.empty(q_lat.shape, dtype=torch.float32, device=q_lat.device) if need_q else None
        d_lat = torch.zeros(latent.shape, dtype=torch.float32, device=latent.device) if need_l else None
        d_W = torch.zeros(W_UV.shape, dtype=torch.float32, device=W_UV.device) if need_w else None
        # on the GPU the element-wise step and the scatter-add are this library's kernels (one pass each); the
        # same arithmetic in framework operations serves the host-side test of this function
        fused = q_lat.is_cuda and indices.shape[1] % 8 == 0
        idx32 = indices.to(torch.int32).contiguous()
        qp32 = q_pos.to(torch.int32).contiguous()
        for t0 in range(0, L, fctx.q_chunk):
            t1 = min(t0 + fctx.q_chunk, L)
            idx = indices[t0:t1].long()
            valid = (idx >= 0) & (idx <= q_pos[t0:t1].long().view(-1, 1))
            idx = idx.clamp(min=0)
            qc = q_lat[t0:t1].detach().to(cdt)
            g = d_out[t0:t1].to(cdt)
            cc = ctx[t0:t1]
            sel = lat[idx]                                                   # [c,K,576]
            s = torch.einsum("thd,tkd->thk", qc, sel)                        # raw scores
            if need_w:
                d_W += torch.einsum("thv,thl->hvl", g, cc.to(cdt)).float()
            d_ctx = torch.einsum("thv,hvl->thl", g, Wc)                      # [c,H,512]
            d_p = torch.einsum("thl,tkl->thk", d_ctx, sel[..., :512])
            delta = (d_ctx.float() * cc.float()).sum(-1)
            if fused:
                p, d_s = K.sparse_attn_bwd_pointwise(s.contiguous(), d_p.contiguous(), lse[t0:t1].contiguous(),
                                                     delta.contiguous(), idx32[t0:t1], qp32[t0:t1], scale)
            else:
                lse_c = lse[t0:t1].unsqueeze(-1)
                p = torch.exp(s.float() * scale - lse_c)
                p = torch.where(valid.unsqueeze(1) & torch.isfinite(lse_c), p, torch.zeros_like(p))
                d_s = (p * (d_p.float() - delta.unsqueeze(-1)) * scale).to(cdt)
                p = p.to(cdt)
            if need_q:
                d_q[t0:t1] = torch.einsum("thk,tkd->thd", d_s, sel).float()
            if need_l:
                d_sel = torch.einsum("thk,thd->tkd", d_s, qc)
                d_sel_v = torch.einsum("thk,thl->tkl", p, d_ctx)
                if fused:
                    K.scatter_add_latent_rows(d_lat, d_sel.contiguous(), d_sel_v.contiguous(), idx32[t0:t1], qp32[t0:t1])
                else:
                    d_sel = d_sel.float()
                    d_sel[..., :512] += d_sel_v.float()
                    d_lat.index_add_(0, idx.reshape(-1), d_sel.reshape(-1, d_sel.shape[-1]))
        return (None if d_q is None else d_q.to(q_lat.dtype), None if d_lat is None else d_lat.to(latent.dtype),
                None if d_W is None else d_W.to(W_UV.dtype), None, None, None, None)


def sparse_attend_absorbed_chunked(q_lat, latent, W_UV, indices, *, d_c: int, sm_scale: float, cu_seqlens=None,
                                   q_chunk: int = 512, checkpoint: bool = True, q_global_pos=None) -> torch.Tensor:
    """Sparse MLA attention in the absorbed latent space followed by the W_UV up-projection;
    [Lq, H, Dv].  Nothing of size [chunk, K, 576] is materialised in the forward pass, so checkpoint is
    accepted and ignored; under autograd the op is differentiable in q_lat, latent and W_UV, and q_chunk
    bounds the [chunk, K, 576] gather of the backward pass (see _SparseAttendAbsorbed)."""
    if d_c != 512:
        raise B200DSAError("d_c must be 512")
    L = q_lat.shape[0]
    if q_global_pos is not None:
        q_pos = q_global_pos
    elif cu_seqlens is not None:
        q_pos = prepare_ks_ke(cu_seqlens)[1] - 1
    else:
        q_pos = torch.arange(L, device=q_lat.device)
    if torch.is_grad_enabled() and (q_lat.requires_grad or latent.requires_grad or W_UV.requires_grad):
        return _SparseAttendAbsorbed.apply(q_lat, latent, W_UV, indices, q_pos, float(sm_scale), int(q_chunk))
    # bf16 context straight from the attention kernel, then the per-head up-projection on tensor cores
    ctx, _ = sparse_attend_latent(q_lat, latent, indices, sm_scale=sm_scale, q_pos=q_pos, ctx_dtype=torch.bfloat16)
    return _up_project(ctx, W_UV)


def patch_opendsa() -> None:
    """Rebind the reference's names to these implementations (the OpenDSA package must be importable)."""
    import opendsa.modeling.dsa_attention as att
    import opendsa.ops as ops
    for mod in (att, ops):
        mod.indexer_select_topk = indexer_select_topk
        mod.sparse_attend_absorbed_chunked = sparse_attend_absorbed_chunked
