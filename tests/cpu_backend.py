"""CPU stand-in for transarch_b200.kernels, built on the oracle.  TEST ONLY: it lets the
host-side orchestration of the key-sharded decode step (shard arithmetic, wire layouts,
collectives, merge order) run on gloo ranks without a GPU.  The shipped package never
imports it."""
import torch

from oracle import dsa_oracle as O

WIRE_ROW = 516
NEG_INF = float("-inf")


def quant_q_fold_weights(q, w, fold, *, q_fp8=None, weights=None):
    T, H, D = q.shape
    a, b = O.quant_q_fold_weights(q.float(), w, fold)
    q_fp8.copy_(a); weights.copy_(b)
    return q_fp8, weights


def indexer_paged_fp8_logits(q_fp8, weights, cache, page_size, context_lens, block_table, *, next_n=1,
                             max_cols=None, out_scale=1.0, out=None, fill=True):
    res = O.paged_indexer_logits(q_fp8.float(), cache, weights, context_lens, block_table, page_size, max_cols,
                                 out_scale)
    out.copy_(res)
    return out


def topk_select(scores, k, *, col_begin=None, col_end=None, keep_pos_inf=False, pos_map=None, page_table=None,
                page_size=0, row_pos_offset=None, sorted=True, return_values=False, out=None, out_values=None,
                seg_cols=0, seg_stride=0, n_cols=None, row_stride=None, n_rows=None, pos_map_stride=None):
    flat = scores.reshape(-1)
    n_rows = scores.shape[0] if n_rows is None else n_rows
    n_cols = scores.shape[1] if n_cols is None else n_cols
    row_stride = scores.stride(0) if row_stride is None else row_stride
    pm = pos_map.reshape(-1) if pos_map is not None else None
    pms = pos_map_stride if pos_map_stride is not None else (pos_map.stride(0) if pos_map is not None else 0)
    cols = torch.arange(n_cols)
    off = (cols // seg_cols) * seg_stride + cols % seg_cols if seg_cols > 0 else cols
    for r in range(n_rows):
        v = flat[r * row_stride + off].clone()
        lo = int(col_begin[r]) if col_begin is not None else 0
        hi = int(col_end[r]) if col_end is not None else n_cols
        ok = (cols >= lo) & (cols < hi) & ~torch.isnan(v) & (v > NEG_INF)
        if not keep_pos_inf:
            ok &= v < float("inf")
        pos = pm[r * pms + off] if pm is not None else cols.to(torch.int32)
        if row_pos_offset is not None:
            pos = pos + int(row_pos_offset[r])
        cand = torch.nonzero(ok).flatten()
        # descending score, ties by ascending output position
        order = sorted_by(v[cand], pos[cand])
        pick = cand[order][:k]
        out[r].fill_(-1)
        out[r, :pick.numel()] = pos[pick].to(torch.int32)
        if out_values is not None:
            out_values[r].fill_(NEG_INF)
            out_values[r, :pick.numel()] = v[pick]
    return (out, out_values) if out_values is not None else out


def sorted_by(vals, pos):
    idx = torch.argsort(pos.long(), stable=True)
    idx2 = torch.argsort(vals[idx], descending=True, stable=True)
    return idx[idx2]


def sparse_mla_decode(q, kv, indices, sm_scale, *, kv_row_base=None, q_pos=None, pos_lo=0, pos_hi=2 ** 31 - 1,
                      n_idx_item=None, ctx=None, lse=None, q_pos_bias=0):
    n = q.shape[0]
    for b in range(n):
        idx = indices[b].long()
        keep = (idx >= pos_lo) & (idx < pos_hi) & (idx >= 0)
        if q_pos is not None:
            keep &= idx <= int(q_pos[b]) + q_pos_bias
        rows = (idx - pos_lo + (int(kv_row_base[b]) if kv_row_base is not None else 0))
        local = torch.where(keep, rows, torch.full_like(rows, -1)).to(torch.int32).view(1, -1)
        c, l = O.sparse_attend_latent(q[b:b + 1], kv, local, d_c=512, sm_scale=sm_scale,
                                      q_pos=torch.tensor([kv.shape[0]]))
        ctx[b].copy_(c[0]); lse[b].copy_(l[0])
    return ctx, lse


def lse_prescale(ctx, lse, lse_max, wire):
    w = torch.where(torch.isfinite(lse), torch.exp(lse - lse_max), torch.zeros_like(lse)).reshape(-1, 1)
    wire.zero_()
    wire[:, :512] = ctx.reshape(-1, 512) * w
    wire[:, 512] = w[:, 0]
    return wire


def lse_finalize(wire, lse_max, ctx_out, lse_out):
    den = wire[:, 512].reshape(lse_max.shape)
    ctx_out.copy_((wire[:, :512] / wire[:, 512:513].clamp_min(1e-38)).reshape(ctx_out.shape))
    ctx_out[den == 0] = 0
    lse_out.copy_(torch.where(den > 0, lse_max + torch.log(den), torch.full_like(den, NEG_INF)))
    return ctx_out, lse_out


def lse_prescale_norm(ctx, lse_all, my_part, out_bf16, lse_out):
    m = lse_all.max(0).values
    ms = torch.where(torch.isfinite(m), m, torch.zeros_like(m))
    w = torch.where(torch.isfinite(lse_all), torch.exp(lse_all - ms), torch.zeros_like(lse_all))
    den = w.sum(0)
    share = torch.where(den > 0, w[my_part] / den.clamp_min(1e-38), torch.zeros_like(den))
    out_bf16.copy_((ctx * share.unsqueeze(-1)).to(torch.bfloat16))
    lse_out.copy_(torch.where(den > 0, ms + torch.log(den), torch.full_like(den, NEG_INF)))
    return out_bf16, lse_out
