"""Fused decode selection (indexer epilogue collects the candidates, one exact select kernel after
it) against the unfused pair of calls on the same inputs: identical logits, identical index sets,
identical order when sorted; ragged / short / empty rows, ties, several query rows per request,
position offsets, and the no-logits mode."""
import pytest
import torch

from oracle import dsa_oracle as O

pytestmark = pytest.mark.gpu
P = 64


def _state(seed, ctxs, next_n=1):
    from transarch_b200.workloads import make_decode_state
    st = make_decode_state(len(ctxs), ctxs, page_size=P, seed=seed)
    g = torch.Generator().manual_seed(seed)
    rows = len(ctxs) * next_n
    q = torch.randn(rows, 64, 128, generator=g).bfloat16().cuda()
    w = (torch.randn(rows, 64, generator=g) / 8).cuda()
    return st, q, w


def _unfused(K, q_fp8, wf, st, row_ctx, k, next_n=1, off=None, sorted_=False):
    logits = K.indexer_paged_fp8_logits(q_fp8, wf, st.k_cache, P, row_ctx, st.block_table, next_n=next_n,
                                        max_cols=st.local_len)
    idx, val = K.topk_select(logits, k, col_end=row_ctx, row_pos_offset=off, sorted=sorted_, return_values=True)
    return logits, idx, val


@pytest.mark.parametrize("ctxs,k", [([131072, 70000, 9000, 2048, 2047, 300, 1, 0, 40000], 2048),
                                     ([8192 + 37 * i for i in range(64)], 2048),
                                     ([20000, 33000, 128, 129], 512),
                                     ([5000] * 7, 64)])
def test_fused_equals_unfused(ctxs, k):
    from transarch_b200 import _lib, kernels as K
    st, q, w = _state(len(ctxs) + k, ctxs)
    q_fp8, wf = K.quant_q_fold_weights(q, w, 128 ** -0.5)
    ref_logits, ref_idx, ref_val = _unfused(K, q_fp8, wf, st, st.context_lens, k)
    scratch = K.fused_scratch(len(ctxs), q.device)
    logits = torch.full_like(ref_logits, float("nan"))
    for rep in range(3):                                        # the scratch is re-armed by every call
        idx, val = K.indexer_paged_fp8_topk(q_fp8, wf, st.k_cache, P, st.context_lens, st.block_table, k, scratch,
                                            max_cols=st.local_len, logits=logits,
                                            out_values=torch.empty(len(ctxs), k, device="cuda"))
        assert torch.equal(torch.sort(idx, 1).values, torch.sort(ref_idx, 1).values), rep
        assert torch.equal(torch.sort(val, 1).values, torch.sort(ref_val, 1).values)
        assert (scratch[1] == 0).all()
    for b, c in enumerate(ctxs):                                 # the by-product logits are the plain kernel's
        assert torch.equal(logits[b, :c], ref_logits[b, :c])
    # sorted output: same order as the unfused sorted selection
    s_idx = K.indexer_paged_fp8_topk(q_fp8, wf, st.k_cache, P, st.context_lens, st.block_table, k, scratch,
                                     max_cols=st.local_len, logits=logits, sorted=True)
    assert torch.equal(s_idx, K.topk_select(ref_logits, k, col_end=st.context_lens, sorted=True))
    # no logits at all: the lists alone decide (and are provably complete here)
    n_idx = K.indexer_paged_fp8_topk(q_fp8, wf, st.k_cache, P, st.context_lens, st.block_table, k, scratch,
                                     max_cols=st.local_len, keep_logits=False)
    assert _lib.read_status(q.device) == 0
    assert torch.equal(torch.sort(n_idx, 1).values, torch.sort(ref_idx, 1).values)


def test_fused_against_oracle_with_offsets_and_two_rows_per_request():
    from transarch_b200 import _lib, kernels as K
    ctxs, next_n, k = [3000, 9000, 700], 2, 256
    st, q, w = _state(5, ctxs, next_n)
    q_fp8, wf = K.quant_q_fold_weights(q, w, 128 ** -0.5)
    row_ctx = (st.context_lens.view(-1, 1) - next_n + torch.arange(next_n, device="cuda", dtype=torch.int32).view(1, -1) + 1)
    row_ctx = row_ctx.reshape(-1).contiguous()
    off = (torch.arange(len(ctxs) * next_n, dtype=torch.int32, device="cuda") * 100000).contiguous()
    scratch = K.fused_scratch(row_ctx.numel(), q.device)
    idx = K.indexer_paged_fp8_topk(q_fp8, wf, st.k_cache, P, row_ctx, st.block_table, k, scratch, next_n=next_n,
                                   max_cols=st.local_len, row_pos_offset=off, sorted=True).cpu()
    assert _lib.read_status(q.device) == 0
    keys = O.unpack_paged_fp8_cache(st.k_cache.cpu(), P)
    for r in range(row_ctx.numel()):
        b, n = r // next_n, int(row_ctx[r])
        kb = O.gather_request_keys(keys, st.block_table[b].cpu(), n)
        sc = O.indexer_scores(q_fp8[r:r + 1].cpu().float(), kb, wf[r:r + 1].cpu(), 1.0)
        ref = O.topk_rows(sc, k)
        got = idx[r:r + 1] - int(off[r])
        got[idx[r:r + 1] < 0] = -1
        O.assert_selection_parity(got, ref, sc, 1e-3, what=f"row {r}")


def test_fused_ties_fall_back_to_the_logits():
    """All scores equal (zero queries): every key passes any floor, the lists overflow, and the rows are
    selected from the logits: lowest positions win.  Without logits the call reports it (status 3)."""
    from transarch_b200 import _lib, kernels as K
    ctxs, k = [30000, 9000], 2048
    st, q, w = _state(6, ctxs)
    q_fp8, wf = K.quant_q_fold_weights(torch.zeros_like(q), w, 128 ** -0.5)
    scratch = K.fused_scratch(2, q.device)
    idx = K.indexer_paged_fp8_topk(q_fp8, wf, st.k_cache, P, st.context_lens, st.block_table, k, scratch,
                                   max_cols=st.local_len, sorted=True)
    assert _lib.read_status(q.device) == 0
    assert torch.equal(idx[0].cpu(), torch.arange(k, dtype=torch.int32))
    assert torch.equal(idx[1].cpu(), torch.arange(k, dtype=torch.int32))
    K.indexer_paged_fp8_topk(q_fp8, wf, st.k_cache, P, st.context_lens, st.block_table, k, scratch,
                             max_cols=st.local_len, keep_logits=False)
    torch.cuda.synchronize()
    assert _lib.read_status(q.device) == 3
    assert (scratch[1] == 0).all()


def test_fused_skewed_scores_still_exact():
    """Scores that drift along the row (later keys score higher, as recency does in real caches): the
    floor a CTA takes from the head of its share is then too low or too high; whatever the lists hold,
    the result must equal the unfused selection."""
    from transarch_b200 import kernels as K
    ctxs, k = [131072, 65536, 50000], 2048
    st, q, w = _state(8, ctxs)
    # scale the cached keys of later pages up: rewrite the per-token scales in place
    cache = st.k_cache.view(-1, P * 132)
    for b, c in enumerate(ctxs):
        pages = st.block_table[b, : (c + P - 1) // P].long()
        ramp = torch.linspace(0.2, 3.0, pages.numel(), device="cuda").view(-1, 1)
        sc = cache[pages, P * 128:].contiguous().view(torch.float32) * ramp
        cache[pages, P * 128:] = sc.contiguous().view(torch.uint8)
    q_fp8, wf = K.quant_q_fold_weights(q, w.abs(), 128 ** -0.5)
    ref_logits, ref_idx, _ = _unfused(K, q_fp8, wf, st, st.context_lens, k)
    scratch = K.fused_scratch(len(ctxs), q.device)
    idx = K.indexer_paged_fp8_topk(q_fp8, wf, st.k_cache, P, st.context_lens, st.block_table, k, scratch,
                                   max_cols=st.local_len)
    assert torch.equal(torch.sort(idx, 1).values, torch.sort(ref_idx, 1).values)
