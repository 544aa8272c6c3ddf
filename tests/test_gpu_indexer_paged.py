"""tcgen05 paged FP8 indexer and bf16 block-list indexer against the oracle."""
import pytest
import torch

from oracle import dsa_oracle as O

pytestmark = pytest.mark.gpu

FP8_RTOL = 1e-2   # stated tolerance for FP8 scores (relative, see oracle.rel_err)
BF16_RTOL = 2e-3  # stated tolerance for bf16 scores


def make_paged_case(seed, ctxs, P, extra_pages=3):
    g = torch.Generator().manual_seed(seed)
    ks = [torch.randn(c, 128, generator=g) for c in ctxs]
    qs = [O.quant_fp8_rows(k) for k in ks]
    n_pages = sum((c + P - 1) // P for c in ctxs) + extra_pages
    cache, table = O.pack_paged_fp8_cache([a for a, _ in qs], [b for _, b in qs], P, n_pages, g)
    B = len(ctxs)
    q = torch.randn(B, 64, 128, generator=g)
    w = torch.randn(B, 64, generator=g) / 8
    q_fp8, wf = O.quant_q_fold_weights(q, w, 128 ** -0.5)
    return q_fp8, wf, cache, table, torch.tensor(ctxs, dtype=torch.int32)


@pytest.mark.parametrize("P", [64, 32, 128])
@pytest.mark.parametrize("ctxs", [[130, 64, 1, 257, 4096], [8192, 5000, 12345]])
def test_paged_fp8_logits(ctxs, P):
    from transarch_b200 import _lib, kernels as K
    q_fp8, wf, cache, table, lens = make_paged_case(len(ctxs) * 7 + P, ctxs, P)
    max_cols = table.shape[1] * P
    ref = O.paged_indexer_logits(q_fp8.float(), cache, wf, lens, table, P, max_cols, 1.0)
    out = K.indexer_paged_fp8_logits(q_fp8.cuda(), wf.cuda(), cache.cuda(), P, lens.cuda(), table.cuda())
    assert _lib.read_status(out.device) == 0
    out = out.cpu()
    assert torch.equal(torch.isfinite(out), torch.isfinite(ref))
    # fp8 x fp8 products are exact in fp32; only the summation order differs
    assert O.rel_err(out, ref) < 1e-4
    assert O.rel_err(out, ref) < FP8_RTOL


def test_paged_fp8_zero_context_and_next_n():
    from transarch_b200 import _lib, kernels as K
    P = 64
    q_fp8, wf, cache, table, lens = make_paged_case(99, [300, 200], P)
    # next_n = 2: rows (b, n) share request b's table; draft token n sees ctx-1+n keys
    q2 = q_fp8.repeat_interleave(2, 0).contiguous()
    w2 = wf.repeat_interleave(2, 0).contiguous()
    lens2 = torch.tensor([299, 300, 0, 200], dtype=torch.int32)
    out = K.indexer_paged_fp8_logits(q2.cuda(), w2.cuda(), cache.cuda(), P, lens2.cuda(), table.cuda(),
                                     next_n=2).cpu()
    ref = O.paged_indexer_logits(q_fp8.float(), cache, wf, lens, table, P, out.shape[1], 1.0)
    assert O.rel_err(out[1], ref[0]) < 1e-4 and O.rel_err(out[3], ref[1]) < 1e-4
    assert torch.isinf(out[0, 299:]).all() and O.rel_err(out[0, :299], ref[0, :299]) < 1e-4
    assert torch.isinf(out[2]).all()
    assert _lib.read_status(torch.device("cuda", 0)) == 0


def test_blocklist_bf16_logits():
    from transarch_b200 import _lib, kernels as K
    g = torch.Generator().manual_seed(8)
    T, S, m = 9, 128 * 37 + 50, 12
    q = torch.randn(T, 64, 128, generator=g).bfloat16()
    k = torch.randn(S, 128, generator=g).bfloat16()
    w = torch.randn(T, 64, generator=g) / 8
    nb = (S + 127) // 128
    lists = torch.stack([torch.randperm(nb, generator=g)[:m] for _ in range(T)]).to(torch.int32)
    nblk = torch.randint(1, m + 1, (T,), generator=g)
    nblk[0] = m
    lists[0, 3] = nb - 1                       # tail block: rows beyond S must come out masked
    for t in range(T):
        lists[t, nblk[t]:] = -1
    row_cols = (nblk * 128).to(torch.int32)
    ke = torch.randint(S // 2, S + 1, (T,), generator=g, dtype=torch.int32)
    ke[0] = S
    ks = torch.randint(0, S // 4, (T,), generator=g, dtype=torch.int32)
    out = K.indexer_blocklist_bf16_logits(q.cuda(), w.cuda(), k.cuda(), lists.cuda(), row_cols.cuda(),
                                          pos_lo=ks.cuda(), pos_hi=ke.cuda(), out_scale=128 ** -0.5)
    assert _lib.read_status(out.device) == 0
    out = out.cpu()
    full = O.indexer_scores(q, k, w, 128 ** -0.5)
    ref = torch.full_like(out, float("-inf"))
    for t in range(T):
        for j in range(int(nblk[t])):
            b = int(lists[t, j])
            pos = torch.arange(b * 128, (b + 1) * 128)
            ok = (pos >= ks[t]) & (pos < ke[t]) & (pos < S)
            ref[t, j * 128:(j + 1) * 128][ok] = full[t, pos[ok]]
    assert torch.equal(torch.isfinite(out), torch.isfinite(ref))
    assert O.rel_err(out, ref) < BF16_RTOL


def test_flat_prefill_groups_of_four_queries_match_the_per_query_kernel():
    """The prefill kernel (four queries per key tile) against the per-query block-list kernel on packed
    documents with ragged intervals, a row count that is not a multiple of four, empty rows and key counts
    that are not a multiple of 128: identical -inf pattern, scores equal up to fp32 summation order."""
    from transarch_b200 import _lib, kernels as K
    g = torch.Generator().manual_seed(91)
    T, S = 203, 5000 + 37
    q = torch.randn(T, 64, 128, generator=g).bfloat16().cuda()
    k = torch.randn(S, 128, generator=g).bfloat16().cuda()
    w = (torch.randn(T, 64, generator=g) / 8).cuda()
    lo = torch.randint(0, 3000, (T,), generator=g, dtype=torch.int32)
    hi = (lo + torch.randint(1, 2000, (T,), generator=g, dtype=torch.int32)).clamp(max=S)
    hi[5] = lo[5]                                             # an empty interval
    lo[6], hi[6] = 0, S                                       # the whole key range
    lo, hi = lo.cuda(), hi.cuda()
    col0 = (lo >> 7) << 7
    row_cols = ((((hi + 127) >> 7) << 7) - col0).clamp(min=0).contiguous()
    cols = (S + 127) // 128 * 128
    ref = K.indexer_blocklist_bf16_logits(q, w, k, None, row_cols, pos_lo=lo, pos_hi=hi, out_scale=0.5, max_cols=cols)
    got = K.indexer_flat_bf16_logits(q, w, k, lo, hi, row_cols, cols, out_scale=0.5)
    assert _lib.read_status(q.device) == 0
    assert torch.equal(torch.isinf(got), torch.isinf(ref))
    fin = torch.isfinite(ref)
    assert (got[fin] - ref[fin]).abs().max() < 1e-5 * ref[fin].abs().max()
    # and against the oracle on a few rows
    for r in (0, 6, 100, 202):
        sc = O.indexer_scores(q[r:r + 1].cpu().float(), k.cpu().float(), w[r:r + 1].cpu(), 0.5)[0]
        a, b = int(lo[r]), int(hi[r])
        c0 = int(col0[r])
        assert O.rel_err(got[r, a - c0:b - c0].cpu().view(1, -1), sc[a:b].view(1, -1)) < 2e-3


def test_routed_flat_kernel_and_gather_kernel():
    """The two kernels of the routed prefill by themselves: eight gathered heads with 32 queries per key tile
    (row count not a multiple of 32, two documents, a query without keys), and all-head scores on per-query
    candidate lists with missing (-1), out-of-range and masked entries."""
    from transarch_b200 import _lib, kernels as K
    g = torch.Generator().manual_seed(77)
    T, N = 75, 1500
    k = torch.randn(N, 128, generator=g).bfloat16()
    q8 = torch.randn(T, 8, 128, generator=g).bfloat16()
    w8 = torch.randn(T, 8, generator=g) / 4
    ke = torch.randint(1, N + 1, (T,), generator=g, dtype=torch.int32)
    ks = torch.zeros(T, dtype=torch.int32)
    ks[40:] = torch.minimum(torch.full((T - 40,), 700, dtype=torch.int32), ke[40:] - 1)
    ke[7] = ks[7]                                                     # no visible key at all
    col0 = (ks >> 7) << 7
    row_cols = ((((ke + 127) >> 7) << 7) - col0).clamp(min=0)
    cols = ((N + 127) // 128) * 128
    out = K.indexer_flat_bf16_logits_routed(q8.cuda(), w8.cuda(), k.cuda(), ks.cuda(), ke.cuda(), row_cols.cuda(), cols,
                                            out_scale=0.25).cpu()
    ref = O.mask_interval(O.indexer_scores(q8.float(), k.float(), w8, 0.25), ks.long(), ke.long())
    for t in range(T):
        n = int(row_cols[t])
        got = out[t, :n]
        want = ref[t, int(col0[t]):int(col0[t]) + n]
        want = torch.cat([want, torch.full((n - want.numel(),), float("-inf"))])
        fin = torch.isfinite(want)
        assert torch.equal(torch.isfinite(got), fin), t
        if fin.any():
            assert O.rel_err(got[fin], want[fin]) < 2e-3, t
    # gather kernel
    q = torch.randn(T, 64, 128, generator=g).bfloat16()
    w = torch.randn(T, 64, generator=g) / 8
    n_cand = 300
    cand = torch.randint(0, N, (T, n_cand), generator=g, dtype=torch.int32)
    cand[:, 17] = -1
    cand[3, 40] = N + 5                                               # beyond the keys: dropped, not read
    cand[5, 200:] = -1
    got = K.indexer_gather_bf16_logits(q.cuda(), w.cuda(), k.cuda(), cand.cuda(), pos_lo=ks.cuda(), pos_hi=ke.cuda(),
                                       out_scale=0.5).cpu()
    full = O.mask_interval(O.indexer_scores(q.float(), k.float(), w, 0.5), ks.long(), ke.long())
    okc = (cand >= 0) & (cand < N)
    want = torch.gather(full, 1, cand.clamp(0, N - 1).long())
    want = torch.where(okc, want, torch.full_like(want, float("-inf")))
    fin = torch.isfinite(want)
    assert torch.equal(torch.isfinite(got), fin)
    assert O.rel_err(got[fin], want[fin]) < 2e-3
    assert _lib.read_status(torch.device("cuda")) == 0
