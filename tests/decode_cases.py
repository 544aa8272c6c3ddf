"""Shared builders for the decode-step tests: a global (unsharded) seeded problem on the CPU and
its split into position shards, each packed as a rank would hold it."""
import torch

from oracle import dsa_oracle as O


def make_global_problem(seed, ctxs, H=128, P=64):
    g = torch.Generator().manual_seed(seed)
    B = len(ctxs)
    keys = [torch.randn(c, 128, generator=g) for c in ctxs]
    kq = [O.quant_fp8_rows(k) for k in keys]
    kv = [(0.5 * torch.randn(c, 576, generator=g)).bfloat16() for c in ctxs]
    q_idx = torch.randn(B, 64, 128, generator=g).bfloat16()
    w = (torch.randn(B, 64, generator=g) / 8).float()
    q_lat = torch.randn(B, H, 576, generator=g).bfloat16()
    return dict(ctxs=list(ctxs), kq=kq, kv=kv, q_idx=q_idx, w=w, q_lat=q_lat, P=P, H=H, gen=g)


def shard_state(prob, rank, world, shard_len, device):
    """Pack rank's position range [rank*shard_len, (rank+1)*shard_len) of every request."""
    P = prob["P"]
    lo = rank * shard_len if world > 1 else 0
    hi = lo + shard_len
    kq_l, sc_l, kv_rows, base, local = [], [], [], [], []
    row = 0
    for (kq, sc), kv in zip(prob["kq"], prob["kv"]):
        a, b = min(lo, kq.shape[0]), min(hi, kq.shape[0])
        kq_l.append(kq[a:b]); sc_l.append(sc[a:b])
        base.append(row)
        kv_rows.append(kv[a:b])
        row += b - a
        local.append(b - a)
    n_pages = sum((n + P - 1) // P for n in local) + 2
    gen = torch.Generator().manual_seed(1234 + rank)
    nonempty = [i for i, n in enumerate(local) if n > 0]
    cache, table = O.pack_paged_fp8_cache([k if k.shape[0] else torch.zeros(0, 128).to(torch.float8_e4m3fn) for k in kq_l],
                                          sc_l, P, n_pages, gen)
    if table.shape[1] == 0:
        table = torch.full((len(local), 1), -1, dtype=torch.int32)
    kv_cat = torch.cat(kv_rows + [torch.zeros(1, 576, dtype=torch.bfloat16)])
    return dict(cache=cache.to(device), table=table.to(device),
                lens=torch.tensor(prob["ctxs"], dtype=torch.int32, device=device),
                local=torch.tensor(local, dtype=torch.int32, device=device),
                kv=kv_cat.to(device), base=torch.tensor(base, dtype=torch.int64, device=device))


def oracle_decode(prob, topk, index_scale, attn_scale):
    """Reference result of the whole step on the unsharded problem (fp32 on the dequantised
    FP8 keys and on the quantised queries the kernels see)."""
    B = len(prob["ctxs"])
    q_fp8, wf = O.quant_q_fold_weights(prob["q_idx"].float(), prob["w"], index_scale)
    idx_all, score_all, ctx_all, lse_all = [], [], [], []
    for b in range(B):
        kq, sc = prob["kq"][b]
        kb = kq.float() * sc.unsqueeze(-1)
        s = O.indexer_scores(q_fp8[b:b + 1].float(), kb, wf[b:b + 1], 1.0)
        idx = O.topk_rows(s, topk)
        c, l = O.sparse_attend_latent(prob["q_lat"][b:b + 1], prob["kv"][b], idx, d_c=512, sm_scale=attn_scale,
                                      q_pos=torch.tensor([prob["ctxs"][b] - 1]))
        idx_all.append(idx); score_all.append(s); ctx_all.append(c); lse_all.append(l)
    return torch.cat(idx_all), score_all, torch.cat(ctx_all), torch.cat(lse_all)
