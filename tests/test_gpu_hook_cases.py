"""The vLLM-facing hook on the cases the reference's glue handles (indexers.py:388-581): the
"ue8m0" scale format, buffers narrower than the requested top-k, a stage-1 shortlist shorter than
the final top-k, padded (mixed-length) decode batches, per-row context lengths as vLLM 0.22 hands
them over, and the registered torch op itself."""
import pytest
import torch

from oracle import dsa_oracle as O

pytestmark = pytest.mark.gpu
P = 64


def _paged(seed, ctxs, ue8m0=False, spare=8):
    g = torch.Generator().manual_seed(seed)
    ks = [torch.randn(c, 128, generator=g).bfloat16().float() for c in ctxs]
    qs = [O.quant_fp8_rows(k, ue8m0=ue8m0) for k in ks]
    n_pages = sum((c + P - 1) // P for c in ctxs) + spare
    cache, table = O.pack_paged_fp8_cache([a for a, _ in qs], [b for _, b in qs], P, n_pages, g)
    return g, ks, qs, cache, table


def _dequant(qs, b):
    return qs[b][0].float() * qs[b][1].unsqueeze(-1)


@pytest.mark.parametrize("ue8m0", [False, True])
def test_quantisers_match_oracle_bitwise(ue8m0):
    """q quantisation + weight folding and the k-cache insert, both scale formats, bit for bit."""
    from transarch_b200 import _lib, kernels as K
    g = torch.Generator().manual_seed(90 + int(ue8m0))
    q = (torch.randn(41, 64, 128, generator=g) * torch.rand(41, 64, 1, generator=g) * 4).bfloat16()
    q[3, 5] = 0                                              # an all-zero head: the scale floor
    q[4, 6] = 448.0 / 1024                                   # amax/448 an exact power of two
    w = torch.randn(41, 64, generator=g) / 8
    q_fp8, wf = K.quant_q_fold_weights(q.cuda(), w.cuda(), 0.125, ue8m0=ue8m0)
    rq, rw = O.quant_q_fold_weights(q.float(), w, 0.125, ue8m0=ue8m0)
    assert torch.equal(q_fp8.cpu().view(torch.uint8), rq.view(torch.uint8))
    assert torch.allclose(wf.cpu(), rw, rtol=1e-6, atol=0)
    if ue8m0:                                                # every folded scale is a power of two
        sc = (wf.cpu() / (w * 0.125)).double()
        m, _ = torch.frexp(sc[w.abs() > 1e-3])
        assert ((m - 0.5).abs() < 1e-5).all()
    # keys into cache slots
    n = 300
    k = (torch.randn(n, 128, generator=g) * torch.rand(n, 1, generator=g) * 3).bfloat16()
    k[7] = 0
    n_pages = 8
    cache = torch.zeros(n_pages, P * 132, dtype=torch.uint8, device="cuda")
    slots = torch.randperm(n_pages * P, generator=g)[:n].to(torch.int64)
    slots[11] = -1                                           # a padding token is skipped
    K.indexer_k_quant_and_cache(k.cuda(), cache, slots.cuda(), P, "ue8m0" if ue8m0 else None)
    assert _lib.read_status(cache.device) == 0
    kq, sc = O.quant_fp8_rows(k.float(), ue8m0=ue8m0)
    c = cache.cpu()
    vals = c[:, :P * 128].reshape(-1, 128)
    scales = c[:, P * 128:].contiguous().view(torch.float32).reshape(-1)
    for t in range(n):
        if slots[t] < 0:
            continue
        assert torch.equal(vals[slots[t]], kq[t].view(torch.uint8)), t
        assert float(scales[slots[t]]) == float(sc[t]), t
    untouched = torch.ones(n_pages * P, dtype=torch.bool)
    untouched[slots[slots >= 0]] = False
    assert (vals[untouched] == 0).all()
    with pytest.raises(Exception):
        K.indexer_k_quant_and_cache(k.cuda(), cache, slots.cuda(), P, "e4m3")


def _decode_setup(seed, ctxs, ue8m0, extra_per_req):
    """A cache holding ctxs[b] keys per request, plus extra_per_req[b] new keys to append."""
    from transarch_b200 import vllm_hook as V
    g, ks, qs, cache, table = _paged(seed, [c + e for c, e in zip(ctxs, extra_per_req)], ue8m0)
    # blank the slots of the keys the hook is going to insert, keep them aside as bf16 inputs
    cache = cache.clone()
    new_k, slots = [], []
    for b, (c, e) in enumerate(zip(ctxs, extra_per_req)):
        for i in range(c, c + e):
            pg, off = int(table[b, i // P]), i % P
            cache[pg, off * 128:(off + 1) * 128] = 0
            cache[pg, P * 128 + off * 4: P * 128 + off * 4 + 4] = 0
            new_k.append(ks[b][i]); slots.append(pg * P + off)
    return g, ks, qs, cache, table, torch.stack(new_k).bfloat16(), torch.tensor(slots, dtype=torch.int64)


@pytest.mark.parametrize("ue8m0", [False, True])
def test_hook_decode_padded_batch_matches_reference_rule(ue8m0):
    """Mixed decode lengths (requires_padding): the reference pads to next_n = max(decode_lens),
    so token j of a request sees seq_len - next_n + j + 1 keys (indexers.py:165-171, :521-551)."""
    from transarch_b200 import _lib, vllm_hook as V
    ctxs, dl = [700, 1500, 130], [2, 1, 2]
    g, ks, qs, cache, table, new_k, slots = _decode_setup(61, ctxs, ue8m0, dl)
    nd, next_n = sum(dl), max(dl)
    q = torch.randn(nd, 64, 128, generator=g)
    w = torch.randn(nd, 64, generator=g) / 8
    q_fp8, wf = O.quant_q_fold_weights(q, w, 128 ** -0.5, 64 ** -0.5, ue8m0=ue8m0)
    seq = torch.tensor([c + e for c, e in zip(ctxs, dl)], dtype=torch.int32)
    buf = torch.full((8, 64), 7, dtype=torch.int32, device="cuda")
    md = V.IndexerMetadata(slot_mapping=slots.cuda(), num_decodes=3, num_decode_tokens=nd,
                           decode=V.DecodeMetadata(seq_lens=seq.cuda(), block_table=table.cuda(),
                                                   decode_lens=torch.tensor(dl).cuda(), requires_padding=True))
    op = V.BaselineSparseAttnIndexer(cache.view(-1, P, 1, 132).cuda(), 128, "ue8m0" if ue8m0 else None, 64, 128,
                                     1600, 4096, buf)
    out = op.forward_cuda(torch.empty(nd, 16, device="cuda"), q_fp8.cuda(), new_k.cuda(), wf.cuda(),
                          attn_metadata=md)
    assert out is buf and _lib.read_status(buf.device) == 0
    t = 0
    for b, d in enumerate(dl):
        kd = _dequant(qs, b)
        for j in range(d):
            n_vis = int(seq[b]) - next_n + j + 1
            sc = O.indexer_scores(q_fp8[t:t + 1].float(), kd[:n_vis], wf[t:t + 1], 1.0)
            O.assert_selection_parity(buf[t:t + 1].cpu(), O.topk_rows(sc, 64), sc, 1e-3, what=f"token {t}")
            t += 1
    assert (buf[nd:] == 7).all()


def test_hook_narrow_buffer_short_table_and_short_stage1():
    """Shapes the reference handles by writing only the columns it has (indexers.py:511-513, :575):
    a block table shorter than topk_tokens keys, and a stage-1 shortlist shorter than topk_tokens."""
    from transarch_b200 import _lib, vllm_hook as V
    ctxs = [100, 128]
    g, ks, qs, cache, table = _paged(62, ctxs)
    table = table[:, :2].contiguous()                         # 2 pages = 128 keys < topk_tokens = 256
    q = torch.randn(2, 64, 128, generator=g)
    w = torch.randn(2, 64, generator=g) / 8
    q_fp8, wf = O.quant_q_fold_weights(q, w, 128 ** -0.5, 64 ** -0.5)
    hq = O.qnorm_head_topk(q, 8)
    seq = torch.tensor(ctxs, dtype=torch.int32)
    no_new = torch.full((2,), -1, dtype=torch.int64)          # nothing to insert this step
    for stage1, topk in ((8192, 256), (16, 64)):
        buf = torch.full((4, 256), 7, dtype=torch.int32, device="cuda")
        md = V.IndexerMetadata(slot_mapping=no_new.cuda(), num_decodes=2, num_decode_tokens=2,
                               decode=V.DecodeMetadata(seq_lens=seq.cuda(), block_table=table.cuda()))
        op = V.MiSASparseAttnIndexer(cache.view(-1, P, 1, 132).cuda(), 128, None, 8, 8, True, 128, stage1, topk, 128,
                                     4096, 4096, buf)
        op.forward_cuda(torch.empty(2, 16, device="cuda"), q_fp8.cuda(), torch.zeros(2, 128).cuda(), wf.cuda(),
                        hq.cuda(), attn_metadata=md)
        assert _lib.read_status(buf.device) == 0
        res = buf.cpu()
        for b, c in enumerate(ctxs):
            ref, full, st1 = _two_stage(q_fp8[b:b + 1].float(), wf[b:b + 1], hq[b:b + 1], _dequant(qs, b)[:c],
                                        stage1, min(topk, 256))
            got = res[b][res[b] >= 0]
            assert got.numel() == int((ref >= 0).sum())
            assert set(got.tolist()) == set(ref[ref >= 0].tolist())
        assert (res[2:] == 7).all()


def _two_stage(q8f, wf, hidx, kd, s1, k):
    qh, wh = O.gather_heads(q8f, wf, hidx)
    st1 = O.indexer_scores(qh, kd, wh, 1.0)
    c1 = torch.topk(st1, min(s1, kd.shape[0]), dim=-1).indices[0]
    full = O.indexer_scores(q8f, kd, wf, 1.0)
    pick = c1[torch.topk(full[0][c1], min(k, c1.numel())).indices]
    ref = torch.full((1, k), -1, dtype=torch.int32)
    ref[0, :pick.numel()] = pick.to(torch.int32)
    return ref, full, st1


def test_adapter_for_per_row_context_lengths_and_registered_op():
    """vLLM 0.22's layer signature with seq_lens [B, next_n] (its multi-token path), and the same
    call through the registered torch op with the metadata taken from a forward-context dictionary."""
    from transarch_b200 import _lib, vllm_hook as V
    ctxs, next_n = [900, 333], 2
    g, ks, qs, cache, table, new_k, slots = _decode_setup(63, ctxs, True, [next_n] * 2)
    nd = 2 * next_n
    q = torch.randn(nd, 64, 128, generator=g)
    w = torch.randn(nd, 64, generator=g) / 8
    q_fp8, wf = O.quant_q_fold_weights(q, w, 128 ** -0.5, 64 ** -0.5, ue8m0=True)
    total = torch.tensor([c + next_n for c in ctxs], dtype=torch.int32)
    per_row = total.view(-1, 1) - next_n + torch.arange(next_n, dtype=torch.int32).view(1, -1) + 1
    buf = torch.full((nd, 128), 7, dtype=torch.int32, device="cuda")
    md = V.IndexerMetadata(slot_mapping=slots.cuda(), num_decodes=2, num_decode_tokens=nd,
                           decode=V.DecodeMetadata(seq_lens=per_row.cuda(), block_table=table.cuda()))
    op = V.SparseAttnIndexer022(cache.view(-1, P, 1, 132).cuda(), 128, "ue8m0", 128, 128, 1024, 4096, buf)
    out = op.forward_cuda(torch.empty(nd, 16, device="cuda"), q_fp8.cuda(), new_k.cuda(), wf.cuda(),
                          attn_metadata=md)
    assert out is buf and _lib.read_status(buf.device) == 0
    t = 0
    for b in range(2):
        kd = _dequant(qs, b)
        for j in range(next_n):
            sc = O.indexer_scores(q_fp8[t:t + 1].float(), kd[:int(per_row[b, j])], wf[t:t + 1], 1.0)
            O.assert_selection_parity(buf[t:t + 1].cpu(), O.topk_rows(sc, 128), sc, 1e-3, what=f"row {t}")
            t += 1
    first = buf.clone()

    # the metadata as vLLM keeps it: a dictionary keyed by the cache's layer name
    args = (torch.empty(nd, 16, device="cuda"), "layer0.k_cache", cache.view(-1, P, 1, 132).cuda(), q_fp8.cuda(),
            new_k.cuda(), wf.cuda(), 128, "ue8m0", 128, 128, 1024, 4096)
    buf2 = torch.full_like(buf, 7)
    V.misa_sparse_attn_indexer(*args[:6], None, 128, "ue8m0", 64, 64, True, None, 128, 128, 128, 1024, 4096, buf2,
                               attn_metadata={"layer0.k_cache": md}, use_misa=False)
    assert torch.equal(buf2, first)
    # and through the registered torch op (the reference's torch.ops.vllm.* call), which finds the
    # metadata in vLLM's forward context, when such a context can be set up outside an engine
    ns = getattr(torch.ops, V.register_ops())
    ctx_mgr = None
    if V.HAVE_VLLM:
        try:
            from vllm.config import VllmConfig
            from vllm.forward_context import set_forward_context
            ctx_mgr = set_forward_context({"layer0.k_cache": md}, VllmConfig())
        except Exception:  # noqa: BLE001 - vLLM refuses a bare config here: the dictionary path above stands
            ctx_mgr = None
    if ctx_mgr is not None:
        buf3 = torch.full_like(buf, 7)
        with ctx_mgr:
            ns.baseline_sparse_attn_indexer(*args, buf3)
        assert torch.equal(buf3, first)
    else:
        # no forward context in scope: the op must behave as a dummy / profiling run (buffer untouched)
        buf3 = torch.full_like(buf, 7)
        ns.baseline_sparse_attn_indexer(*args, buf3)
        assert (buf3 == 7).all()
