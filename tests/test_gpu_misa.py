"""MISA routers, routed two-stage logits and the vLLM-style hook against the oracle."""
import pytest
import torch

from oracle import dsa_oracle as O

pytestmark = pytest.mark.gpu


def _paged(seed, ctxs, P=64):
    g = torch.Generator().manual_seed(seed)
    ks = [torch.randn(c, 128, generator=g) for c in ctxs]
    qs = [O.quant_fp8_rows(k) for k in ks]
    n_pages = sum((c + P - 1) // P for c in ctxs) + 3
    cache, table = O.pack_paged_fp8_cache([a for a, _ in qs], [b for _, b in qs], P, n_pages, g)
    return g, qs, cache, table


def test_routers_match_oracle():
    from transarch_b200 import kernels as K
    g = torch.Generator().manual_seed(30)
    T = 19
    q = torch.randn(T, 64, 128, generator=g).bfloat16()
    w = torch.randn(T, 64, generator=g) / 8
    # q-norm
    wo, hi = K.router_qnorm_topk(q.cuda(), w.cuda(), 8)
    ref = O.qnorm_head_topk(q, 8)
    assert torch.equal(torch.sort(hi.cpu().long(), 1).values, torch.sort(ref, 1).values)
    assert torch.equal(wo.cpu(), torch.zeros(T, 64).scatter_(1, ref, torch.gather(w, 1, ref)))
    # block score
    kblk = torch.randn(37, 128, generator=g)
    lo = torch.randint(0, 5, (T,), generator=g, dtype=torch.int32)
    hi_b = torch.randint(6, 38, (T,), generator=g, dtype=torch.int32)
    wo, hidx, sc = K.router_block_score_topk(q.cuda(), w.cuda(), kblk.cuda(), lo.cuda(), hi_b.cuda(), 8,
                                             return_scores=True)
    ref_sc = O.misa_block_head_scores(q, kblk, w, lo.long(), hi_b.long())
    assert torch.allclose(sc.cpu(), ref_sc, rtol=2e-4, atol=1e-5)
    ref_idx = torch.topk(ref_sc, 8, dim=-1).indices
    assert torch.equal(torch.sort(hidx.cpu().long(), 1).values, torch.sort(ref_idx, 1).values)
    # linear router (no reference code; oracle restatement)
    x = torch.randn(T, 7168, generator=g).bfloat16()
    W = (torch.randn(7168, 64, generator=g) * 7168 ** -0.5).bfloat16()
    wo, hidx, lg = K.router_linear_topk_softmax(x.cuda(), W.cuda(), 8, return_logits=True)
    ridx, rw, rlog = O.linear_router_topk_softmax(x, W, 8)
    assert torch.allclose(lg.cpu(), rlog, rtol=1e-3, atol=1e-3)
    assert torch.equal(torch.sort(hidx.cpu().long(), 1).values, torch.sort(ridx, 1).values)
    dense = torch.zeros(T, 64).scatter_(1, ridx, rw)
    assert torch.allclose(wo.cpu(), dense, rtol=2e-3, atol=1e-4)
    assert torch.allclose(wo.cpu().sum(1), torch.ones(T), atol=1e-5)


def test_pooling_matches_oracle():
    from transarch_b200 import kernels as K
    g = torch.Generator().manual_seed(31)
    k = torch.randn(1000, 128, generator=g).bfloat16()
    p16, p32 = K.block_mean_pool(k.cuda(), 128, want_f32=True)
    ref = O.block_mean_pool(k.float(), 128)
    assert torch.allclose(p32.cpu(), ref, rtol=1e-5, atol=1e-6)
    assert (p16.cpu().float() - ref).abs().max() < 4e-3
    _, qs, cache, table = _paged(32, [300, 64, 1000])
    lens = torch.tensor([300, 64, 1000], dtype=torch.int32)
    pooled = K.paged_mean_pool_fp8(cache.cuda(), 64, lens.cuda(), table.cuda(), 128, 8).cpu()
    for b, c in enumerate([300, 64, 1000]):
        kd = qs[b][0].float() * qs[b][1].unsqueeze(-1)
        ref = O.block_mean_pool(kd, 128)
        assert torch.allclose(pooled[b, :ref.shape[0]], ref, rtol=1e-5, atol=1e-6)
        assert (pooled[b, ref.shape[0]:] == 0).all()


def test_pooled_key_cache_follows_the_cache_bit_exactly():
    """Incremental pooled-key maintenance: after every growth step (one token, a few tokens, across a
    block boundary, a slot taken over by a shorter request) the kept means equal pooling the whole
    cache again, bit for bit, and feed misa_page_mqa_logits to the same result."""
    from transarch_b200 import kernels as K, misa as M
    ctx_final = [700, 64, 1000]
    g, qs, cache, table = _paged(36, ctx_final)
    cache, table = cache.cuda(), table.cuda()
    state = K.PooledKeyCache(3, 8, 128, "cuda")
    steps = [[300, 10, 500], [301, 11, 501], [304, 12, 640], [513, 64, 641], [513, 64, 1000]]
    for lens in steps:
        lens_t = torch.tensor(lens, dtype=torch.int32, device="cuda")
        got = state.update(cache, 64, lens_t, table)
        ref = K.paged_mean_pool_fp8(cache, 64, lens_t, table, 128, 8)
        assert torch.equal(got, ref), lens
    # slot 0 is taken over by a new, shorter request (same pages here, other length): rebuilt and cleared
    state.reset(torch.tensor([0], device="cuda"))
    lens_t = torch.tensor([130, 64, 1000], dtype=torch.int32, device="cuda")
    got = state.update(cache, 64, lens_t, table)
    assert torch.equal(got, K.paged_mean_pool_fp8(cache, 64, lens_t, table, 128, 8))
    assert (got[0, 2:] == 0).all()
    from transarch_b200 import _lib
    assert _lib.read_status(torch.device("cuda")) == 0
    # the routed decode logits are the same with the kept means
    q = torch.randn(3, 1, 64, 128, generator=g)
    q_fp8 = q.cuda().to(torch.float8_e4m3fn)
    w = (torch.randn(3, 64, generator=g) / 8).cuda()
    a = M.misa_page_mqa_logits(q_fp8, cache.view(-1, 64, 1, 132), w, None, lens_t, table, 1024, 8, False, 256, 128)
    b = M.misa_page_mqa_logits(q_fp8, cache.view(-1, 64, 1, 132), w, None, lens_t, table, 1024, 8, False, 256, 128,
                               pooled=got)
    # the stage-1 candidates come out in no particular order: compare them as sorted (position, logit) pairs
    for x, y in ((a, b),):
        ox, oy = torch.sort(x[1], dim=1).indices, torch.sort(y[1], dim=1).indices
        assert torch.equal(torch.gather(x[1], 1, ox), torch.gather(y[1], 1, oy))
        assert torch.equal(torch.gather(x[0], 1, ox), torch.gather(y[0], 1, oy))


@pytest.mark.parametrize("use_qnorm,s1,two_docs", [(True, 512, False), (False, 512, False), (True, 2048, False),
                                                   (True, 384, True)])
def test_misa_mqa_logits_prefill(use_qnorm, s1, two_docs):
    """s1 = 512 / 384 of 3000 keys: the two-stage form (eight gathered heads, 32 queries per key tile, then
    all heads on the gathered candidates); s1 = 2048: the one-pass form.  two_docs: the later queries belong
    to a second document that starts inside a key tile."""
    from transarch_b200 import misa as M
    g = torch.Generator().manual_seed(33)
    Mq, N = 40 if two_docs else 24, 3000
    k = torch.randn(N, 128, generator=g)
    kq, sc = O.quant_fp8_rows(k)
    q = torch.randn(Mq, 64, 128, generator=g)
    w = torch.randn(Mq, 64, generator=g) / 8
    q_fp8, wf = O.quant_q_fold_weights(q, w, 128 ** -0.5, 64 ** -0.5)
    ke = torch.arange(N - Mq, N, dtype=torch.int32) + 1
    ks = torch.zeros(Mq, dtype=torch.int32)
    if two_docs:
        ks[Mq // 2:] = 1111
    hidx = O.qnorm_head_topk(q, 8) if use_qnorm else None
    logits, cand = M.misa_mqa_logits(q_fp8.cuda(), (kq.cuda(), sc.cuda()), wf.cuda(),
                                     None if hidx is None else hidx.cuda(), ks.cuda(), ke.cuda(), use_qnorm, 8, s1,
                                     k_block_size=128)
    kb = (kq.float() * sc.unsqueeze(-1)).bfloat16().float()
    qf = q_fp8.float()
    if not use_qnorm:
        pooled = O.block_mean_pool(kb.bfloat16(), 128).float()
        hs = O.misa_block_head_scores(qf, pooled, wf, ks.long() // 128, (ke.long() + 127) // 128)
        hidx = torch.topk(hs, 8, dim=-1).indices
    ref_logits, ref_cand = O.misa_mqa_logits(qf, kb, wf, hidx, ks.long(), ke.long(), s1)
    q8, w8 = O.gather_heads(qf, wf, hidx)
    s1_scores = O.mask_interval(O.indexer_scores(q8, kb, w8, 1.0), ks.long(), ke.long())
    O.assert_selection_parity(cand.cpu(), ref_cand, s1_scores, 2e-3, what="stage-1 candidates")
    full = O.mask_interval(O.indexer_scores(qf, kb, wf, 1.0), ks.long(), ke.long())
    got = torch.gather(full, 1, cand.cpu().clamp(min=0).long())
    ok = cand.cpu() >= 0
    assert O.rel_err(logits.cpu()[ok], got[ok]) < 2e-3


def _two_stage_ref(q8f, wf, hidx, kd, s1, k):
    """Oracle two-stage selection of one query row: (picks int32 [1,k] -1 padded, all-head scores
    [1,n], routed stage-1 scores [1,n])."""
    qh, wh = O.gather_heads(q8f, wf, hidx)
    st1 = O.indexer_scores(qh, kd, wh, 1.0)
    c1 = torch.topk(st1, min(s1, kd.shape[0]), dim=-1).indices[0]
    full = O.indexer_scores(q8f, kd, wf, 1.0)
    pick = c1[torch.topk(full[0][c1], min(k, c1.numel())).indices]
    ref = torch.full((1, k), -1, dtype=torch.int32)
    ref[0, :pick.numel()] = pick.to(torch.int32)
    return ref, full, st1


def test_misa_page_logits_and_hook_decode_prefill():
    from transarch_b200 import _lib, misa as M, vllm_hook as V
    ctxs = [700, 1500, 130]
    g, qs, cache, table = _paged(34, ctxs)
    B = len(ctxs)
    q = torch.randn(B, 64, 128, generator=g)
    w = torch.randn(B, 64, generator=g) / 8
    q_fp8, wf = O.quant_q_fold_weights(q, w, 128 ** -0.5, 64 ** -0.5)
    lens = torch.tensor(ctxs, dtype=torch.int32)
    cache4 = cache.view(cache.shape[0], 64, 1, 132).cuda()
    hidx = O.qnorm_head_topk(q, 8)
    logits, cand = M.misa_page_mqa_logits(q_fp8.view(B, 1, 64, 128).cuda(), cache4, wf.cuda(), hidx.cuda(),
                                          lens.cuda(), table.cuda(), 1536, 8, True, 256)
    final = M.misa_final_topk(logits, cand, 64).cpu()
    for b, c in enumerate(ctxs):
        kd = qs[b][0].float() * qs[b][1].unsqueeze(-1)
        ref, full, st1 = _two_stage_ref(q_fp8[b:b + 1].float(), wf[b:b + 1], hidx[b:b + 1], kd, 256, 64)
        O.assert_selection_parity(final[b:b + 1], ref, full, 1e-3, stage1_scores=st1, stage1_k=256,
                                  what=f"paged two-stage, request {b}")

    # ---- hook, decode step: new key appended, then selection over the cache
    P = 64
    buf = torch.full((8, 64), 7, dtype=torch.int32, device="cuda")
    new_k = torch.randn(B, 128, generator=g).bfloat16()
    slots = torch.tensor([int(table[b, c // P]) * P + c % P for b, c in enumerate(ctxs)], dtype=torch.int64)
    cache_dev = cache.clone().view(cache.shape[0], 64, 1, 132).cuda()
    md = V.IndexerMetadata(slot_mapping=slots.cuda(), num_decodes=B, num_decode_tokens=B,
                           decode=V.DecodeMetadata(seq_lens=(lens + 1).cuda(), block_table=table.cuda()))
    op = V.BaselineSparseAttnIndexer(cache_dev, 128, None, 64, 128, 1536, 4096, buf)
    out = op.forward_cuda(torch.empty(B, 16, device="cuda"), q_fp8.cuda(), new_k.cuda(), wf.cuda(),
                          attn_metadata=md)
    assert out is buf and _lib.read_status(buf.device) == 0
    nkq, nsc = O.quant_fp8_rows(new_k.float())
    for b, c in enumerate(ctxs):
        kd = torch.cat([qs[b][0].float() * qs[b][1].unsqueeze(-1), (nkq[b].float() * nsc[b]).view(1, -1)])
        sc = O.indexer_scores(q_fp8[b:b + 1].float(), kd, wf[b:b + 1], 1.0)
        O.assert_selection_parity(buf[b:b + 1].cpu(), O.topk_rows(sc, 64), sc, 1e-3, what=f"hook decode {b}")
    assert (buf[B:] == 7).all()                                # rows of other tokens untouched

    # ---- hook, prefill chunk with two requests (MISA, q-norm heads)
    ctx2 = [200, 333]
    T = sum(ctx2)
    g2, qs2, cache2, table2 = _paged(35, [0, 0])                 # empty cache, keys arrive through the hook
    n_pages = 12
    cache2 = torch.zeros(n_pages, 64 * 132, dtype=torch.uint8)
    table2 = torch.tensor([[0, 1, 2, 3, -1, -1], [4, 5, 6, 7, 8, 9]], dtype=torch.int32)
    kf = torch.randn(T, 128, generator=g2).bfloat16()
    qf = torch.randn(T, 64, 128, generator=g2)
    wq = torch.randn(T, 64, generator=g2) / 8
    q8, w8 = O.quant_q_fold_weights(qf, wq, 128 ** -0.5, 64 ** -0.5)
    slot, ks, ke = [], [], []
    for r, c in enumerate(ctx2):
        off = sum(ctx2[:r])
        for i in range(c):
            slot.append(int(table2[r, i // 64]) * 64 + i % 64)
            ks.append(off); ke.append(off + i + 1)
    chunk = V.PrefillChunk(0, T, table2.cuda(), torch.tensor([0, 200, 533], dtype=torch.int32).cuda(),
                           torch.tensor(ks, dtype=torch.int32).cuda(), torch.tensor(ke, dtype=torch.int32).cuda(), T)
    md = V.IndexerMetadata(slot_mapping=torch.tensor(slot).cuda(), num_prefills=2,
                           prefill=V.PrefillMetadata([chunk]))
    buf2 = torch.zeros(T, 32, dtype=torch.int32, device="cuda")
    hq = O.qnorm_head_topk(qf, 8)
    op2 = V.MiSASparseAttnIndexer(cache2.view(n_pages, 64, 1, 132).cuda(), 128, None, 8, 8, True, 128, 128, 32, 128,
                                  384, 4096, buf2)
    op2.forward_cuda(torch.empty(T, 16, device="cuda"), q8.cuda(), kf.cuda(), w8.cuda(), hq.cuda(), attn_metadata=md)
    kq_all, sc_all = O.quant_fp8_rows(kf.float())
    kd_all = kq_all.float() * sc_all.unsqueeze(-1)
    res = buf2.cpu()
    for t in range(T):
        r = 0 if t < 200 else 1
        off = 0 if r == 0 else 200
        kd = kd_all[off: ke[t]]
        ref, full, st1 = _two_stage_ref(q8[t:t + 1].float(), w8[t:t + 1], hq[t:t + 1], kd, 128, 32)
        assert int((res[t] >= 0).sum()) == int((ref >= 0).sum())
        O.assert_selection_parity(res[t:t + 1], ref, full, 1e-3, stage1_scores=st1, stage1_k=128,
                                  what=f"hook prefill token {t}")


def test_single_pass_gated_and_full_scores():
    """The one-pass (all heads, routed heads) pair equals two separate passes bit for bit: a pass
    with the original weights, and a pass with zero weights on the dropped heads."""
    from transarch_b200 import _lib, kernels as K
    from transarch_b200.misa import gate_weights_by_heads
    from transarch_b200.opendsa_ops import identity_block_lists
    ctxs = [700, 64, 2049, 1]
    g, qs, cache, table = _paged(11, ctxs)
    B = len(ctxs)
    q = torch.randn(B, 64, 128, generator=g)
    w = torch.randn(B, 64, generator=g) / 8
    heads = torch.stack([torch.randperm(64, generator=g)[:8] for _ in range(B)]).to(torch.int32)
    heads[0, 0], heads[1, 0] = 63, 0                                   # both ends of the mask word
    q8, wf = K.quant_q_fold_weights(q.cuda().bfloat16(), w.cuda(), 128 ** -0.5)
    lens = torch.tensor(ctxs, dtype=torch.int32).cuda()
    mask = K.head_mask_from_indices(heads.cuda())
    for b in range(B):
        want = sum(1 << int(h) for h in set(heads[b].tolist()))
        assert (int(mask[b]) & (2 ** 64 - 1)) == want
    kw = dict(max_cols=2112)
    full, gated = K.indexer_paged_fp8_logits(q8, wf, cache.cuda(), 64, lens, table.cuda(), head_mask=mask, **kw)
    full_ref = K.indexer_paged_fp8_logits(q8, wf, cache.cuda(), 64, lens, table.cuda(), **kw)
    gated_ref = K.indexer_paged_fp8_logits(q8, gate_weights_by_heads(wf, heads.cuda()), cache.cuda(), 64, lens,
                                           table.cuda(), **kw)
    assert torch.equal(full, full_ref) and torch.equal(gated, gated_ref)
    assert not torch.equal(full[:, :1], gated[:, :1])
    # bf16 block-list form
    N = 1000
    k = torch.randn(N, 128, generator=g).bfloat16().cuda()
    T = 5
    qb = torch.randn(T, 64, 128, generator=g).bfloat16().cuda()
    wb = (torch.randn(T, 64, generator=g) / 8).cuda()
    hb = torch.stack([torch.randperm(64, generator=g)[:8] for _ in range(T)]).to(torch.int32).cuda()
    ks = torch.zeros(T, dtype=torch.int32).cuda()
    ke = torch.tensor([1000, 300, 129, 128, 1], dtype=torch.int32).cuda()
    bl, row_cols = identity_block_lists(ks.long(), ke.long(), N)
    f2, g2 = K.indexer_blocklist_bf16_logits(qb, wb, k, bl, row_cols, pos_lo=ks, pos_hi=ke,
                                             head_mask=K.head_mask_from_indices(hb))
    f2_ref = K.indexer_blocklist_bf16_logits(qb, wb, k, bl, row_cols, pos_lo=ks, pos_hi=ke)
    g2_ref = K.indexer_blocklist_bf16_logits(qb, gate_weights_by_heads(wb, hb), k, bl, row_cols, pos_lo=ks, pos_hi=ke)
    assert torch.equal(f2, f2_ref) and torch.equal(g2, g2_ref)
    assert _lib.read_status(full.device) == 0


def test_misa_prefill_two_stage_edge_cases():
    """Two-stage routed prefill where the pieces do not line up: five kept heads (padded to eight with zero
    weights), a stage-1 budget that is no multiple of 128, queries that see fewer keys than the budget (their
    candidate rows end in -1 / -inf), and a query count that is no multiple of 32."""
    from transarch_b200 import misa as M
    g = torch.Generator().manual_seed(41)
    Mq, N, s1 = 45, 2600, 1000
    k = torch.randn(N, 128, generator=g)
    kq, sc = O.quant_fp8_rows(k)
    q = torch.randn(Mq, 64, 128, generator=g)
    w = torch.randn(Mq, 64, generator=g) / 8
    q_fp8, wf = O.quant_q_fold_weights(q, w, 128 ** -0.5, 64 ** -0.5)
    ke = torch.randint(1, N + 1, (Mq,), generator=g, dtype=torch.int32)
    ke[:5] = torch.tensor([1, 7, 130, 999, 1001], dtype=torch.int32)      # fewer keys than the budget
    ks = torch.zeros(Mq, dtype=torch.int32)
    hidx = O.qnorm_head_topk(q, 5)
    logits, cand = M.misa_mqa_logits(q_fp8.cuda(), (kq.cuda(), sc.cuda()), wf.cuda(), hidx.cuda(), ks.cuda(), ke.cuda(),
                                     True, 5, s1)
    assert logits.shape == (Mq, s1) and cand.shape == (Mq, s1)
    kb = (kq.float() * sc.unsqueeze(-1)).bfloat16().float()
    qf = q_fp8.float()
    q8, w8 = O.gather_heads(qf, wf, hidx)
    s1_scores = O.mask_interval(O.indexer_scores(q8, kb, w8, 1.0), ks.long(), ke.long())
    ref_cand = O.topk_rows(s1_scores, s1)
    O.assert_selection_parity(cand.cpu(), ref_cand, s1_scores, 2e-3, what="stage-1 candidates, five heads")
    n_valid = (cand.cpu() >= 0).sum(1)
    assert torch.equal(n_valid, torch.minimum(ke.long(), torch.tensor(s1)))
    full = O.mask_interval(O.indexer_scores(qf, kb, wf, 1.0), ks.long(), ke.long())
    got = torch.gather(full, 1, cand.cpu().clamp(min=0).long())
    ok = cand.cpu() >= 0
    assert O.rel_err(logits.cpu()[ok], got[ok]) < 2e-3
    assert torch.isinf(logits.cpu()[~ok]).all() and (logits.cpu()[~ok] < 0).all()
