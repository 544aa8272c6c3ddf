"""CPU restatement of the reference's sparse-attention selection path.

TEST INFRASTRUCTURE ONLY (checker + timed CPU baseline); never imported by the
shipped package.  Each function cites the reference lines it follows (paths
relative to the TransArch checkout).  Pinned against the reference itself by
``tests/golden/make_golden.py`` (which imports the reference's OpenDSA ops and
stores their outputs) and ``tests/test_oracle_golden.py``.

Parity status per function:
  * pinned by running the reference: prepare_ks_ke, prepare_ks_ke_cp,
    indexer_scores / indexer_select_topk, sparse_attend_latent
  * restatement of TileLang kernels that cannot run on a CPU (parity pinned only
    through the formula they share with indexer_scores): block_mean_pool,
    misa_block_head_scores, misa_* orchestration, paged variants
  * parity unpinned (no reference code exists): hisa_select_topk,
    linear_router_topk_softmax
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

NEG_INF = float("-inf")


# --------------------------------------------------------------------------- #
# causal intervals
# --------------------------------------------------------------------------- #
def prepare_ks_ke(cu_seqlens: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """[ks, ke) per packed query.  OpenDSA/opendsa/ops/flashkl_warmup.py:41-56."""
    cu = cu_seqlens.to(torch.int64)
    total = int(cu[-1]) if cu.numel() else 0
    t = torch.arange(total, dtype=torch.int64)
    doc = torch.searchsorted(cu, t, right=True) - 1
    ks = cu[doc]
    ke = t + 1
    return ks, ke


def prepare_ks_ke_cp(cu_full: torch.Tensor, q_global_pos: torch.Tensor):
    """Interval per local query at a global position.
    OpenDSA/opendsa/ops/flashkl_warmup.py:235-248."""
    cu = cu_full.to(torch.int64)
    p = q_global_pos.to(torch.int64)
    d = (torch.searchsorted(cu, p, right=True) - 1).clamp(0, cu.numel() - 2)
    return cu[d], p + 1


# --------------------------------------------------------------------------- #
# the indexer's producer: projections, key LayerNorm, RoPE
# --------------------------------------------------------------------------- #
def rope_rotate_half(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x * cos + rotate_half(x) * sin on the last dim (64 rope dims).
    OpenDSA/opendsa/modeling/indexer.py:27-37."""
    half = x.shape[-1] // 2
    rot = torch.cat((-x[..., half:], x[..., :half]), dim=-1)
    return x * cos + rot * sin


def lightning_indexer_forward(h, q_in, cos, sin, state, n_heads: int, head_dim: int = 128, rope_dim: int = 64,
                              ln_eps: float = 1e-5):
    """q = wq(q_in) [B,L,H,d]; k = LayerNorm(wk(h)) [B,L,d]; RoPE on the LAST rope_dim dims of both;
    w = w_proj(h) * H^-0.5.  OpenDSA/opendsa/modeling/indexer.py:64-83.  `state` holds the module's
    parameters under its own names."""
    B, L, _ = h.shape
    q = (q_in.float() @ state["wq.weight"].float().T).view(B, L, n_heads, head_dim)
    k = torch.nn.functional.layer_norm(h.float() @ state["wk.weight"].float().T, (head_dim,),
                                       state["k_norm.weight"].float(), state["k_norm.bias"].float(), ln_eps)
    d0 = head_dim - rope_dim
    q = torch.cat([q[..., :d0], rope_rotate_half(q[..., d0:], cos.unsqueeze(2), sin.unsqueeze(2))], dim=-1)
    k = torch.cat([k[..., :d0], rope_rotate_half(k[..., d0:], cos, sin)], dim=-1)
    w = (h.float() @ state["w_proj.weight"].float().T) * n_heads ** -0.5
    return q, k, w


# --------------------------------------------------------------------------- #
# lightning-indexer score and top-k
# --------------------------------------------------------------------------- #
def indexer_scores(q: torch.Tensor, k: torch.Tensor, w: torch.Tensor,
                   sm_scale: Optional[float] = None, q_chunk: int = 256) -> torch.Tensor:
    """I[t,j] = sm_scale * sum_h w[t,h] * relu(<q[t,h], k[j]>), fp32, unmasked.
    OpenDSA/opendsa/ops/topk_select.py:60-63."""
    q = q.float(); k = k.float(); w = w.float()
    Lq, H, d = q.shape
    sf = sm_scale if sm_scale is not None else d ** -0.5
    out = torch.empty(Lq, k.shape[0], dtype=torch.float32)
    for t0 in range(0, Lq, q_chunk):
        t1 = min(t0 + q_chunk, Lq)
        sh = torch.einsum("thd,jd->thj", q[t0:t1], k)
        sh.relu_()
        sh.mul_(w[t0:t1].unsqueeze(-1))
        out[t0:t1] = sh.sum(1).mul_(sf)
    return out


def mask_interval(scores: torch.Tensor, ks: torch.Tensor, ke: torch.Tensor) -> torch.Tensor:
    """-inf outside [ks, ke).  OpenDSA/opendsa/ops/topk_select.py:64-65."""
    jj = torch.arange(scores.shape[1]).view(1, -1)
    ok = (jj >= ks.view(-1, 1)) & (jj < ke.view(-1, 1))
    return scores.masked_fill(~ok, NEG_INF)


def topk_rows(scores: torch.Tensor, topk: int, keep_pos_inf: bool = False) -> torch.Tensor:
    """Row-wise top-k positions, value-descending, -1 where the pick is not finite.
    OpenDSA/opendsa/ops/topk_select.py:66-71.  keep_pos_inf=True only drops -inf picks
    (needed for force-kept blocks, which carry +inf)."""
    Lq, Lk = scores.shape
    out = torch.full((Lq, topk), -1, dtype=torch.int32)
    k_eff = min(topk, Lk)
    if k_eff == 0:
        return out
    vals, idx = torch.topk(scores, k_eff, dim=-1)
    ok = (vals > NEG_INF) if keep_pos_inf else torch.isfinite(vals)
    out[:, :k_eff] = torch.where(ok, idx.to(torch.int32),
                                 torch.full_like(idx, -1, dtype=torch.int32))
    return out


def indexer_select_topk(index_q, index_k, index_w, cu_seqlens, topk, *,
                        sm_scale_index=None, q_chunk=256, q_global_pos=None) -> torch.Tensor:
    """OpenDSA/opendsa/ops/topk_select.py:30-72."""
    if q_global_pos is None:
        ks, ke = prepare_ks_ke(cu_seqlens)
    else:
        ks, ke = prepare_ks_ke_cp(cu_seqlens, q_global_pos)
    Lq = index_q.shape[0]
    out = torch.full((Lq, topk), -1, dtype=torch.int32)
    for t0 in range(0, Lq, q_chunk):
        t1 = min(t0 + q_chunk, Lq)
        s = indexer_scores(index_q[t0:t1], index_k, index_w[t0:t1], sm_scale_index, q_chunk)
        s = mask_interval(s, ks[t0:t1], ke[t0:t1])
        out[t0:t1] = topk_rows(s, topk)
    return out


# --------------------------------------------------------------------------- #
# sparse MLA attention in the absorbed latent space
# --------------------------------------------------------------------------- #
def sparse_attend_latent(q_lat, latent, indices, *, d_c, sm_scale, q_pos=None):
    """Latent-space context and log-sum-exp per (query, head).

    Follows OpenDSA/opendsa/ops/sparse_mla.py:39-43 and :90 (validity =
    idx>=0 and idx<=q_pos); stops before the W_UV up-projection of :44.
    Fully masked rows give ctx = 0 (:45-47) and lse = -inf.
    Returns (ctx [L,H,d_c] fp32, lse [L,H] fp32)."""
    q = q_lat.float(); lat = latent.float()
    L, H, Dl = q.shape
    if q_pos is None:
        q_pos = torch.arange(L)
    idx = indices.long()
    valid = (idx >= 0) & (idx <= q_pos.view(L, 1).long())
    sel = lat[idx.clamp(min=0)]                                    # [L,K,Dl]
    scores = torch.einsum("thd,tkd->thk", q, sel) * sm_scale
    scores = scores.masked_fill(~valid.view(L, 1, -1), NEG_INF)
    lse = torch.logsumexp(scores, dim=-1)
    probs = torch.nan_to_num(torch.softmax(scores, dim=-1), nan=0.0)
    ctx = torch.einsum("thk,tkl->thl", probs, sel[..., :d_c])
    return ctx, lse


def sparse_attend_absorbed(q_lat, latent, W_UV, indices, *, d_c, sm_scale, q_pos=None):
    """With the up-projection.  OpenDSA/opendsa/ops/sparse_mla.py:26-48."""
    ctx, _ = sparse_attend_latent(q_lat, latent, indices, d_c=d_c, sm_scale=sm_scale, q_pos=q_pos)
    return torch.einsum("thl,hvl->thv", ctx, W_UV.float())


def lse_combine(ctx_parts, lse_parts):
    """Merge per-shard (ctx, lse) partials: out = sum_r ctx_r*exp(lse_r-m) / sum_r exp(lse_r-m)."""
    lse = torch.stack(lse_parts)                                   # [R,L,H]
    m = lse.max(0).values
    m_safe = torch.where(torch.isfinite(m), m, torch.zeros_like(m))
    wgt = torch.exp(lse - m_safe)                                  # exp(-inf)=0
    den = wgt.sum(0)
    num = sum(c * wgt[i].unsqueeze(-1) for i, c in enumerate(ctx_parts))
    out = torch.where(den.unsqueeze(-1) > 0, num / den.clamp_min(1e-38).unsqueeze(-1),
                      torch.zeros_like(num))
    return out, m_safe + torch.log(den)


# --------------------------------------------------------------------------- #
# FP8 key cache (layout the vLLM indexer cache uses)
# --------------------------------------------------------------------------- #
FP8_MAX = 448.0


def pow2_round_up(x: torch.Tensor) -> torch.Tensor:
    """Smallest power of two >= x for positive finite x: exp2(ceil(log2(x))), the "ue8m0" scale
    format, evaluated exactly through frexp (x = m * 2**e with 0.5 <= m < 1)."""
    m, e = torch.frexp(x.float())
    return torch.ldexp(torch.ones_like(m), torch.where(m > 0.5, e, e - 1))


def quant_fp8_rows(x: torch.Tensor, ue8m0: bool = False, eps: float = 1e-4):
    """Per-row e4m3 quantisation, scale = max(amax, eps)/448 (fp32), rounded up to a power of two
    when ue8m0.  Published behaviour of the two third-party vLLM (pinned 0.17.0) quantisers the
    reference calls, neither of which is under the TransArch checkout:
      * keys: ops.indexer_k_quant_and_cache(k, kv_cache, slot_mapping, quant_block_size, scale_fmt)
        at MISA_preprint/misa_vllm_patch_2stage/misa_vllm_patch/indexers.py:454-460, eps = 1e-4,
        ue8m0 when scale_fmt == "ue8m0" (the reference sets it so, misa_deepseek_v2.py:177);
      * queries: per_token_group_quant_fp8(q, 128, use_ue8m0=scale_fmt is not None) at
        misa_deepseek_v2.py:280-285, eps = 1e-10."""
    xf = x.float()
    amax = xf.abs().amax(dim=-1, keepdim=True).clamp_min(eps)
    scale = amax / FP8_MAX
    if ue8m0:
        scale = pow2_round_up(scale)
    q = (xf / scale).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return q, scale.squeeze(-1).contiguous()


def pack_paged_fp8_cache(k_fp8_list, scale_list, page_size: int, num_pages: int,
                         gen: torch.Generator):
    """Scatter per-request FP8 keys into a shuffled paged cache.

    Page layout = page_size*D fp8 bytes followed by page_size fp32 scales, as read at
    MISA_preprint/misa_vllm_patch_2stage/misa_vllm_patch/misa_ops.py:360-372.
    Returns (cache uint8 [num_pages, page_size*(D+4)], block_table int32 [B,max_pages])."""
    D = k_fp8_list[0].shape[1]
    B = len(k_fp8_list)
    need = [(k.shape[0] + page_size - 1) // page_size for k in k_fp8_list]
    assert sum(need) <= num_pages
    perm = torch.randperm(num_pages, generator=gen)
    cache = torch.zeros(num_pages, page_size * (D + 4), dtype=torch.uint8)
    table = torch.full((B, max(need) if need else 0), -1, dtype=torch.int32)
    cur = 0
    for b, (kq, sc) in enumerate(zip(k_fp8_list, scale_list)):
        n = kq.shape[0]
        for p in range(need[b]):
            pg = int(perm[cur]); cur += 1
            table[b, p] = pg
            r0, r1 = p * page_size, min((p + 1) * page_size, n)
            rows = r1 - r0
            cache[pg, : rows * D] = kq[r0:r1].view(torch.uint8).reshape(-1)
            sc_bytes = sc[r0:r1].contiguous().view(torch.uint8).reshape(-1)
            cache[pg, page_size * D: page_size * D + rows * 4] = sc_bytes
    return cache, table


def unpack_paged_fp8_cache(cache: torch.Tensor, page_size: int, D: int = 128):
    """(keys fp32 [num_pages, page_size, D]) = fp8 * scale.
    MISA_preprint/misa_vllm_patch_2stage/misa_vllm_patch/misa_ops.py:360-378."""
    num_pages = cache.shape[0]
    flat = cache.view(num_pages, -1)
    kq = flat[:, : page_size * D].contiguous().view(torch.float8_e4m3fn).view(num_pages, page_size, D)
    sc = flat[:, page_size * D:].contiguous().view(torch.float32).view(num_pages, page_size)
    return kq.float() * sc.unsqueeze(-1)


def gather_request_keys(keys_paged: torch.Tensor, table_row: torch.Tensor, ctx: int):
    """Keys of one request in position order, [ctx, D]."""
    P = keys_paged.shape[1]
    n_pages = (ctx + P - 1) // P
    pages = table_row[:n_pages].long()
    return keys_paged[pages].reshape(n_pages * P, -1)[:ctx]


def paged_indexer_logits(q, cache, w, context_lens, block_table, page_size, max_len,
                         sm_scale: float = 1.0):
    """Decode logits [B, max_len], -inf at and beyond each request's context length.
    Formula of paged_mqa_sparse_head_return_logits
    (MISA_preprint/misa_vllm_patch_2stage/misa_vllm_patch/misa_ops.py:56-159), computed in
    fp32 on exactly the dequantised fp8 values.  q [B,H,D], w [B,H]."""
    B = q.shape[0]
    keys = unpack_paged_fp8_cache(cache, page_size, q.shape[-1])
    out = torch.full((B, max_len), NEG_INF, dtype=torch.float32)
    for b in range(B):
        ctx = int(context_lens[b])
        if ctx == 0:
            continue
        kb = gather_request_keys(keys, block_table[b], ctx)
        out[b, :ctx] = indexer_scores(q[b:b + 1], kb, w[b:b + 1], sm_scale)[0]
    return out


def quant_q_fold_weights(q: torch.Tensor, w: torch.Tensor, sm_scale: float, head_scale: float = 1.0,
                         ue8m0: bool = False):
    """q -> e4m3 per (token, head) with its scale folded into the head weight.
    MISA_preprint/misa_vllm_patch_2stage/misa_vllm_patch/misa_deepseek_v2.py:279-292
    (weights = w * q_scale * softmax_scale * n_head**-0.5; there the n_head factor is
    applied here, in OpenDSA it is already inside w, hence head_scale).  ue8m0 is the
    use_ue8m0 flag of :280-285 (True in the reference, whose scale_fmt is never None)."""
    T_, H, D = q.shape
    q_fp8, q_scale = quant_fp8_rows(q.reshape(T_ * H, D), ue8m0=ue8m0, eps=1e-10)
    weights = w.float() * q_scale.view(T_, H) * (sm_scale * head_scale)
    return q_fp8.view(T_, H, D), weights


# --------------------------------------------------------------------------- #
# block pooling, HISA two-stage selection
# --------------------------------------------------------------------------- #
def block_mean_pool(k: torch.Tensor, block: int) -> torch.Tensor:
    """Mean of each run of `block` rows, the tail divided by its true length; fp32
    accumulate then cast back.  MISA_preprint/.../block_ops.py:685-754."""
    S, D = k.shape
    nb = (S + block - 1) // block
    kf = k.float()
    pad = nb * block - S
    if pad:
        kf = torch.cat([kf, torch.zeros(pad, D)], 0)
    sums = kf.view(nb, block, D).sum(1)
    cnt = torch.full((nb, 1), float(block))
    if pad:
        cnt[-1] = block - pad
    return (sums / cnt).to(k.dtype)


def hisa_block_logits(q, k_blk, w, ks, ke, block, sm_scale=None,
                      keep_first: bool = False, keep_last: bool = True):
    """Stage-1 block scores [T, n_blocks]: indexer formula on pooled keys, -inf outside the
    query's block range, +inf on force-kept blocks
    (mask/keep rule: MISA_preprint/.../block_ops.py:576-666; HISA description
    HISA_COLM_2026/README.md:5-6).  Parity unpinned: the reference ships no HISA code."""
    s = indexer_scores(q, k_blk, w, sm_scale)
    bks = ks // block
    bke = (ke + block - 1) // block
    s = mask_interval(s, bks, bke)
    rows = torch.arange(s.shape[0])
    has = bke > bks
    if keep_last:
        s[rows[has], (bke - 1)[has]] = float("inf")
    if keep_first:
        s[rows[has], bks[has]] = float("inf")
    return s


def hisa_select_topk(q, k, w, ks, ke, *, block=128, block_topk=64, topk=2048,
                     sm_scale=None, keep_first=False, keep_last=True, q_chunk=64,
                     return_blocks=False, blocks=None, return_scores=False):
    """HISA: pool -> block top-m -> token scores inside the chosen blocks -> top-k.
    Returns int32 [T, topk] absolute positions (-1 padded).  Parity unpinned.
    blocks (int32 [T, m], -1 padded): skip stage 1 and run stage 2 inside these blocks (to check
    stage 2 by itself).  return_scores adds the stage-2 scores as a dense [T, S_padded] tensor
    (-inf outside the chosen blocks) for near-tie audits."""
    T_ = q.shape[0]
    S = k.shape[0]
    k_blk = block_mean_pool(k, block)
    nb = k_blk.shape[0]
    out = torch.full((T_, topk), -1, dtype=torch.int32)
    blocks_out = torch.full((T_, block_topk), -1, dtype=torch.int32)
    pad = nb * block - S
    kf = k.float()
    if pad:
        kf = torch.cat([kf, torch.zeros(pad, k.shape[1])], 0)
    given = blocks
    dense = torch.full((T_, nb * block), NEG_INF) if return_scores else None
    for t0 in range(0, T_, q_chunk):
        t1 = min(t0 + q_chunk, T_)
        if given is None:
            bl = hisa_block_logits(q[t0:t1], k_blk, w[t0:t1], ks[t0:t1], ke[t0:t1], block,
                                   sm_scale, keep_first, keep_last)
            blocks = topk_rows(bl, block_topk, keep_pos_inf=True)                   # [c,m] (-1 padded)
        else:
            blocks = given[t0:t1]
        blocks_out[t0:t1] = blocks
        for i in range(t1 - t0):
            t = t0 + i
            bsel = blocks[i][blocks[i] >= 0].long()
            if bsel.numel() == 0:
                continue
            pos = (bsel.view(-1, 1) * block + torch.arange(block).view(1, -1)).reshape(-1)
            sc = indexer_scores(q[t:t + 1], kf[pos], w[t:t + 1], sm_scale)[0]
            ok = (pos >= ks[t]) & (pos < ke[t])
            sc = sc.masked_fill(~ok, NEG_INF)
            if dense is not None:
                dense[t, pos] = sc
            pick = topk_rows(sc.view(1, -1), topk)[0]
            good = pick >= 0
            res = torch.full((topk,), -1, dtype=torch.int32)
            res[good] = pos[pick[good].long()].to(torch.int32)
            out[t] = res
    res = (out,) + ((blocks_out,) if return_blocks else ()) + ((dense,) if return_scores else ())
    return res if len(res) > 1 else out


# --------------------------------------------------------------------------- #
# MISA head routing
# --------------------------------------------------------------------------- #
def qnorm_head_topk(q: torch.Tensor, n_heads_keep: int) -> torch.Tensor:
    """Heads with the largest L2 norm.
    MISA_preprint/misa_vllm_patch_2stage/misa_vllm_patch/misa_deepseek_v2.py:254-266."""
    nrm = q.float().norm(dim=-1)
    return torch.topk(nrm, n_heads_keep, dim=-1, sorted=False).indices


def misa_block_head_scores(q, k_blk, w, bks, bke):
    """QScores[t,h] = sum over the query's pooled blocks of |w[t,h]*relu(<k_blk,q[t,h]>)|.
    MISA_preprint/.../block_ops.py:546-569 (prefill) and :11-98 (decode)."""
    q = q.float(); kb = k_blk.float(); w = w.float()
    s = torch.einsum("thd,jd->thj", q, kb).relu_() * w.unsqueeze(-1)
    jj = torch.arange(kb.shape[0]).view(1, 1, -1)
    ok = (jj >= bks.view(-1, 1, 1)) & (jj < bke.view(-1, 1, 1))
    return (s.abs() * ok).sum(-1)


def linear_router_topk_softmax(x, W_r, n_heads_keep: int):
    """logits = x @ W_r; keep the top heads; weights = softmax over the kept logits.
    No reference code exists for this router (parity unpinned); ties broken by lowest head."""
    logits = x.float() @ W_r.float()
    vals, idx = torch.topk(logits, n_heads_keep, dim=-1)
    return idx, torch.softmax(vals, dim=-1), logits


def gather_heads(q, w, head_idx):
    """MISA_preprint/misa_vllm_patch_2stage/misa_vllm_patch/misa_ops.py:703-705."""
    qi = head_idx.long().unsqueeze(-1).expand(-1, -1, q.shape[-1])
    return torch.gather(q, 1, qi), torch.gather(w, 1, head_idx.long())


def misa_mqa_logits(q, k, w, head_idx, ks, ke, stage1_topk, sm_scale=1.0):
    """Routed prefill: stage-1 logits with the kept heads, stage-1 top candidates,
    stage-2 all-head logits on those candidates.
    MISA_preprint/misa_vllm_patch_2stage/misa_vllm_patch/misa_ops.py:703-713.
    Computed in fp32 (the reference rounds operands to bf16 at :688-690).
    Returns (logits [M, s1], candidate positions int32 [M, s1])."""
    q8, w8 = gather_heads(q.float(), w.float(), head_idx)
    s1 = mask_interval(indexer_scores(q8, k, w8, sm_scale), ks, ke)
    n1 = min(stage1_topk, k.shape[0])
    cand = torch.topk(s1, n1, dim=-1, sorted=False).indices
    full = mask_interval(indexer_scores(q, k, w, sm_scale), ks, ke)
    return torch.gather(full, 1, cand), cand.to(torch.int32)


# --------------------------------------------------------------------------- #
# one request of the decode step, end to end
# --------------------------------------------------------------------------- #
def decode_request_reference(q_idx, w, q_lat, pages, kv, ctx_len: int, topk: int, index_scale: float,
                             attn_scale: float, page_size: int = 64, ue8m0: bool = False):
    """Reference result of one decode request, driven as the reference's ops are driven for decode:
    q quantisation + weight folding (misa_deepseek_v2.py:279-292), dequantised paged keys
    (misa_ops.py:360-378), indexer_select_topk with q_global_pos = ctx_len - 1
    (OpenDSA/opendsa/ops/topk_select.py:30-72) and the latent attention of sparse_mla.py:39-43.
      q_idx [1,64,128], w [1,64], q_lat [1,H,576]; pages uint8 [n_pages, page_size*132] = the request's
      cache pages in position order; kv [>=ctx_len, 576].
    Returns (scores fp32 [1,ctx_len], idx int32 [1,topk], ctx fp32 [1,H,512], lse fp32 [1,H])."""
    q_fp8, wf = quant_q_fold_weights(q_idx.float(), w.float(), index_scale, ue8m0=ue8m0)
    keys = unpack_paged_fp8_cache(pages, page_size).reshape(-1, 128)[:ctx_len]
    scores = indexer_scores(q_fp8.float(), keys, wf, 1.0)
    idx = topk_rows(scores, topk)
    ctx, lse = sparse_attend_latent(q_lat, kv[:ctx_len], idx, d_c=512, sm_scale=attn_scale,
                                    q_pos=torch.tensor([ctx_len - 1]))
    return scores, idx, ctx, lse


def check_decode_request(scores_ref, idx_ref, got_logits, got_idx, got_ctx, got_lse, q_lat, kv, ctx_len: int,
                         attn_scale: float):
    """Compare one request of a decode step with decode_request_reference's result.  Returns a dict of
    measured errors; raises AssertionError when a stated tolerance is missed: FP8 scores 1e-2 relative,
    index sets recall >= 0.999 with only near-tie disagreements, attention 2e-2 (checked on the
    implementation's own picks, so that ties cannot leak into the attention comparison)."""
    res = {}
    if got_logits is not None:
        res["score_rel_err"] = rel_err(got_logits.float().view(1, -1)[:, :ctx_len], scores_ref)
        assert res["score_rel_err"] < 1e-2, res
    res["recall"] = assert_selection_parity(got_idx.view(1, -1), idx_ref, scores_ref, 1e-3, what="decode request")
    c, l = sparse_attend_latent(q_lat, kv[:ctx_len], got_idx.view(1, -1), d_c=512, sm_scale=attn_scale,
                                q_pos=torch.tensor([ctx_len - 1]))
    res["attn_rel_err"] = float((got_ctx.float().view_as(c) - c).abs().max() / c.abs().max().clamp_min(1e-9))
    res["lse_abs_err"] = float((got_lse.float().view_as(l) - l).abs().max())
    assert res["attn_rel_err"] < 2e-2 and res["lse_abs_err"] < 2e-2, res
    return res


# --------------------------------------------------------------------------- #
# metrics
# --------------------------------------------------------------------------- #
def set_recall(pred: torch.Tensor, ref: torch.Tensor) -> float:
    """Mean over rows of |pred ∩ ref| / |ref| on the non-negative entries (rows with an
    empty reference count as 1).  Metric of
    MISA_preprint/misa_vllm_patch_2stage/misa_vllm_patch/test_speed.py:115-126."""
    tot = 0.0
    for p, r in zip(pred.tolist(), ref.tolist()):
        rs = {x for x in r if x >= 0}
        if not rs:
            tot += 1.0 if not any(x >= 0 for x in p) else 0.0
            continue
        ps = {x for x in p if x >= 0}
        tot += len(ps & rs) / len(rs)
    return tot / max(1, pred.shape[0])


def near_tie_audit(pred: torch.Tensor, ref: torch.Tensor, scores: torch.Tensor,
                   rtol: float, stage1_scores: Optional[torch.Tensor] = None,
                   stage1_k: int = 0) -> Tuple[int, int]:
    """Count disagreements and how many of them are NOT near-ties at the k-th score.
    A disagreement (in pred xor ref) is a near-tie when
    |s[i] - s_kth| <= rtol * max(|s_kth|, rms(s_valid)).
    Two-stage selections (a stage-1 shortlist of the stage1_k best stage1_scores, then the top-k of
    `scores` inside it) also excuse a disagreement whose stage-1 score is a near-tie at the
    stage1_k-th stage-1 score: whether it was shortlisted at all was decided by a tie."""
    bad = 0
    total = 0
    for t in range(pred.shape[0]):
        rs = {x for x in ref[t].tolist() if x >= 0}
        ps = {x for x in pred[t].tolist() if x >= 0}
        diff = ps ^ rs
        if not diff:
            continue
        total += len(diff)
        srow = scores[t]
        ref_idx = torch.tensor(sorted(rs), dtype=torch.long)
        kth = srow[ref_idx].min()
        fin = srow[torch.isfinite(srow)]
        tol = rtol * max(float(kth.abs()), float(fin.pow(2).mean().sqrt()))
        kth1 = tol1 = None
        if stage1_scores is not None:
            s1 = stage1_scores[t]
            fin1 = s1[torch.isfinite(s1)]
            if fin1.numel() > stage1_k > 0:
                kth1 = float(torch.topk(fin1, stage1_k).values[-1])
                tol1 = rtol * max(abs(kth1), float(fin1.pow(2).mean().sqrt()))
        for i in diff:
            if abs(float(srow[i]) - float(kth)) <= tol:
                continue
            if kth1 is not None and abs(float(stage1_scores[t][i]) - kth1) <= tol1:
                continue
            bad += 1
    return total, bad


def assert_selection_parity(pred: torch.Tensor, ref: torch.Tensor, scores: torch.Tensor, rtol: float,
                            stage1_scores: Optional[torch.Tensor] = None, stage1_k: int = 0,
                            what: str = "selection") -> float:
    """The acceptance rule for index sets: recall >= 0.999 and every disagreement a near-tie."""
    rec = set_recall(pred, ref)
    total, bad = near_tie_audit(pred, ref, scores, rtol, stage1_scores, stage1_k)
    assert bad == 0, f"{what}: {bad} of {total} disagreements are not near-ties (recall {rec:.5f})"
    assert rec >= 0.999, f"{what}: recall {rec:.5f} < 0.999 ({total} disagreements, all near-ties)"
    return rec


def finite_top(scores: torch.Tensor) -> torch.Tensor:
    """Replace +inf entries (force-kept blocks) by a finite value just above the largest finite score,
    so that a near-tie audit can compute magnitudes without the infinities changing the order."""
    fin = torch.where(torch.isfinite(scores), scores, torch.full_like(scores, NEG_INF))
    top = fin.max(dim=1, keepdim=True).values
    top = torch.where(torch.isfinite(top), top, torch.zeros_like(top))
    return torch.where(torch.isposinf(scores), (top + top.abs() + 1.0).expand_as(scores), scores)


def rel_err(x: torch.Tensor, ref: torch.Tensor, eps: float = 1e-2) -> float:
    """max |x-ref| / max(|ref|, eps*rms(ref)) over finite reference entries."""
    m = torch.isfinite(ref)
    r = ref[m].double(); v = x[m].double()
    if r.numel() == 0:
        return 0.0
    den = torch.maximum(r.abs(), eps * r.pow(2).mean().sqrt().clamp_min(1e-30))
    return float(((v - r).abs() / den).max())
