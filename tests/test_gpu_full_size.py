"""Full-size runs of the benchmark configurations, checked through size-independent properties
(selection threshold property, ownership / range / uniqueness of the picks, split-and-merge
equality of attention) plus oracle spot checks on a few rows."""
import pytest
import torch

from oracle import dsa_oracle as O

pytestmark = pytest.mark.gpu
K_TOP = 2048


def _check_selection(logits, idx, lens, k):
    """Every pick is a valid, distinct column, and no unpicked score beats a picked one."""
    B = logits.shape[0]
    for b in range(B):
        n = int(lens[b])
        got = idx[b][idx[b] >= 0].long()
        assert got.numel() == min(k, n)
        assert int(got.max()) < n and got.unique().numel() == got.numel()
        row = logits[b, :n]
        picked = torch.zeros(n, dtype=torch.bool, device=row.device)
        picked[got] = True
        if got.numel() < n:
            assert row[picked].min() >= row[~picked].max()


def test_config2_ragged_decode_indexer_full_size():
    """Batch 64, ragged contexts uniform in [8K, 32K], FP8 paged keys, top-2048, seed 1."""
    from transarch_b200 import _lib, kernels as K
    from transarch_b200.workloads import make_decode_queries, make_decode_state
    g = torch.Generator().manual_seed(1)
    lens = torch.randint(8192, 32769, (64,), generator=g).tolist()
    st = make_decode_state(64, lens, seed=1)
    q_idx, w, _ = make_decode_queries(64, seed=1)
    q_fp8, wf = K.quant_q_fold_weights(q_idx, w, 128 ** -0.5)
    logits = K.indexer_paged_fp8_logits(q_fp8, wf, st.k_cache, 64, st.context_lens, st.block_table,
                                        max_cols=st.local_len)
    idx = K.topk_select(logits, K_TOP, col_end=st.context_lens, sorted=False)
    idx2 = K.topk_select_split(logits, K_TOP, K.topk_scratch(64, logits.device), col_end=st.context_lens,
                               sorted=False)
    assert _lib.read_status(logits.device) == 0
    _check_selection(logits, idx, st.context_lens, K_TOP)
    assert torch.equal(torch.sort(idx, 1).values, torch.sort(idx2, 1).values)
    # -inf exactly beyond each context (rounded up to the tile the kernel wrote)
    for b in (0, 17, 63):
        assert torch.isfinite(logits[b, :lens[b]]).all() and torch.isinf(logits[b, lens[b]:]).all()
    # against the oracle on EVERY request: scores within the stated FP8 tolerance, index sets audited
    cache_cpu, table_cpu = st.k_cache.cpu(), st.block_table.cpu()
    keys = O.unpack_paged_fp8_cache(cache_cpu, 64)
    q_cpu, w_cpu, idx_cpu, logits_cpu = q_fp8.cpu().float(), wf.cpu(), idx.cpu(), logits.cpu()
    for b in range(64):
        kb = O.gather_request_keys(keys, table_cpu[b], lens[b])
        ref = O.indexer_scores(q_cpu[b:b + 1], kb, w_cpu[b:b + 1], 1.0)
        assert O.rel_err(logits_cpu[b:b + 1, :lens[b]], ref) < 1e-2          # stated FP8 tolerance
        O.assert_selection_parity(idx_cpu[b:b + 1], O.topk_rows(ref, K_TOP), ref, 1e-3, what=f"request {b}")


def test_config5_attention_split_and_merge_full_size():
    """Batch 64, 128 heads, 2048 selected keys each: attending two halves of the selection and
    merging by log-sum-exp equals attending the whole selection."""
    from transarch_b200 import _lib, kernels as K
    g = torch.Generator(device="cuda").manual_seed(4)
    B, rows = 64, 16384
    kv = (0.5 * torch.randn(B * rows, 576, generator=g, device="cuda")).bfloat16()
    q = torch.randn(B, 128, 576, generator=g, device="cuda").bfloat16()
    base = torch.arange(B, dtype=torch.int64, device="cuda") * rows
    idx = torch.stack([torch.randperm(rows, generator=g, device="cuda")[:K_TOP] for _ in range(B)]).to(torch.int32)
    scale = 192 ** -0.5
    full, lse = K.sparse_mla_decode(q, kv, idx, scale, kv_row_base=base)
    full, lse = full.clone(), lse.clone()
    halves = []
    for h in range(2):
        part = idx.clone()
        part[:, (1 - h) * 1024:(2 - h) * 1024] = -1
        c, l = K.sparse_mla_decode(q, kv, part, scale, kv_row_base=base)
        halves.append((c.clone(), l.clone()))
    merged, mlse = K.lse_combine(torch.stack([halves[0][0], halves[1][0]]), torch.stack([halves[0][1], halves[1][1]]))
    assert _lib.read_status(kv.device) == 0
    assert (merged - full).abs().max() < 2e-3 * full.abs().max()
    assert (mlse - lse).abs().max() < 1e-3
    # oracle spot check on two items
    for b in (0, 63):
        c, l = O.sparse_attend_latent(q[b:b + 1].cpu(), kv[b * rows:(b + 1) * rows].cpu(), idx[b:b + 1].cpu(),
                                      d_c=512, sm_scale=scale, q_pos=torch.tensor([rows]))
        assert (full[b].cpu() - c[0]).abs().max() < 2e-2 * c.abs().max()
        assert (lse[b].cpu() - l[0]).abs().max() < 2e-2


def test_config5_decode_step_against_oracle_at_benchmark_size():
    """The benchmarked workload itself: batch 64, context 131072, FP8 paged index keys, top-2048, 128
    heads over 576-wide latent rows, seed 4.  Six sampled requests are compared with the oracle at
    full length: indexer scores, selected index sets (recall and near-tie audit) and attention output."""
    from transarch_b200 import _lib
    from transarch_b200.decode import SparseDecodeStep
    from transarch_b200.workloads import make_decode_queries, make_decode_state
    B, CTX = 64, 131072
    dev = torch.device("cuda")
    st = make_decode_state(B, CTX, page_size=64, seed=4, device=dev)
    step = SparseDecodeStep(B, CTX, page_size=64, topk=K_TOP, n_heads=128, device=dev, ctx_dtype=torch.bfloat16)
    q_idx, w, q_lat = make_decode_queries(B, 128, seed=100, device=dev)
    idx, ctx, lse = step.run(q_idx, w, q_lat, st.k_cache, st.context_lens, st.block_table, st.kv, st.kv_row_base,
                             st.context_lens_local)
    torch.cuda.synchronize()
    assert _lib.read_status(dev) == 0
    _check_selection(step.logits, idx, st.context_lens, K_TOP)           # all 64 rows: threshold property
    for b in (0, 7, 21, 38, 50, 63):
        pages = st.k_cache[st.block_table[b].long()].cpu()
        kv_b = st.kv[b * CTX:(b + 1) * CTX].cpu()
        sc, ref_idx, _, _ = O.decode_request_reference(q_idx[b:b + 1].cpu(), w[b:b + 1].cpu(), q_lat[b:b + 1].cpu(),
                                                       pages, kv_b, CTX, K_TOP, 128 ** -0.5, 192 ** -0.5)
        res = O.check_decode_request(sc, ref_idx, step.logits[b].cpu(), idx[b].cpu(), ctx[b].cpu(), lse[b].cpu(),
                                     q_lat[b:b + 1].cpu(), kv_b, CTX, 192 ** -0.5)
        assert res["recall"] >= 0.999


def test_config3_hisa_long_context_properties():
    """HISA over S = 131072 keys (block 128, top-64 blocks, top-2048); 256 of the 4096 queries of
    the configuration, taken evenly from positions 126976..131071, seed 2."""
    from transarch_b200.hisa import HisaConfig, hisa_select_topk
    from transarch_b200 import kernels as K
    g = torch.Generator(device="cuda").manual_seed(2)
    S, T = 131072, 256
    k = torch.randn(S, 128, generator=g, device="cuda").bfloat16()
    q = torch.randn(T, 64, 128, generator=g, device="cuda").bfloat16()
    w = torch.randn(T, 64, generator=g, device="cuda") / 8
    pos = torch.arange(126976, 131072, 16, device="cuda")
    ks, ke = torch.zeros(T, dtype=torch.int64, device="cuda"), pos + 1
    idx, blocks = hisa_select_topk(q, k, w, ks, ke, HisaConfig(), return_blocks=True)
    assert (blocks >= 0).all() and (blocks[:, 0] == (pos // 128).to(torch.int32)).all()      # last block kept, first
    assert (idx >= 0).all() and (idx.long() < ke.view(-1, 1)).all()
    in_blocks = (idx.view(T, -1, 1) // 128 == blocks.view(T, 1, -1)).any(-1)
    assert in_blocks.all()
    # stage 1 against the oracle on every sampled query: block scores on the pooled keys, audited
    qc, kc, wc, ksc, kec = q.cpu(), k.cpu(), w.cpu(), ks.cpu(), ke.cpu()
    blk_scores = O.hisa_block_logits(qc, O.block_mean_pool(kc, 128), wc, ksc, kec, 128)
    ref_blocks = O.topk_rows(blk_scores, 64, keep_pos_inf=True)
    blk_scores = O.finite_top(blk_scores)               # the forced block's +inf -> just above the row's best
    O.assert_selection_parity(blocks.cpu(), ref_blocks, blk_scores, 2e-3, what="HISA blocks at 128K")
    # stage 2 against the oracle inside the blocks the kernel kept, every sampled query
    ref2, tok_scores = O.hisa_select_topk(qc, kc, wc, ksc, kec, block=128, block_topk=64, topk=2048,
                                          blocks=blocks.cpu(), return_scores=True)
    O.assert_selection_parity(idx.cpu(), ref2, tok_scores, 2e-3, what="HISA tokens at 128K")


def test_config4_misa_linear_router_decode_full_size():
    """Batch 32, context 65536, hidden 7168, top-8 of 64 heads by a linear router with softmax
    weights, FP8 paged keys, top-2048, seed 3."""
    from transarch_b200 import kernels as K, misa as M
    from transarch_b200.workloads import make_decode_queries, make_decode_state
    st = make_decode_state(32, 65536, seed=3)
    q_idx, _, _ = make_decode_queries(32, seed=3)
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(32, 7168, generator=g, device="cuda").bfloat16()
    W_r = (torch.randn(7168, 64, generator=g, device="cuda") * 7168 ** -0.5).bfloat16()
    ones = torch.ones(32, 64, device="cuda")
    q_fp8, fold = K.quant_q_fold_weights(q_idx, ones, 128 ** -0.5)          # fold = q scale * softmax scale
    idx, heads = M.misa_linear_router_decode(x, W_r, q_fp8, fold, st.k_cache, 64, st.context_lens, st.block_table,
                                             8, K_TOP, max_cols=65536)
    ridx, rw, _ = O.linear_router_topk_softmax(x.cpu(), W_r.cpu(), 8)
    assert torch.equal(torch.sort(heads.cpu().long(), 1).values, torch.sort(ridx, 1).values)
    gate = torch.zeros(32, 64).scatter_(1, ridx, rw).cuda() * fold
    logits = K.indexer_paged_fp8_logits(q_fp8, gate.contiguous(), st.k_cache, 64, st.context_lens, st.block_table,
                                        max_cols=65536)
    _check_selection(logits, idx, st.context_lens, K_TOP)
    # against the oracle at full size on four requests: scores (FP8 tolerance) and index sets (audited)
    cache_cpu, table_cpu = st.k_cache.cpu(), st.block_table.cpu()
    keys = O.unpack_paged_fp8_cache(cache_cpu, 64)
    for b in (0, 11, 22, 31):
        kb = O.gather_request_keys(keys, table_cpu[b], 65536)
        ref_s = O.indexer_scores(q_fp8[b:b + 1].cpu().float(), kb, gate[b:b + 1].cpu(), 1.0)
        assert O.rel_err(logits[b:b + 1, :65536].cpu(), ref_s) < 1e-2
        O.assert_selection_parity(idx[b:b + 1].cpu(), O.topk_rows(ref_s, K_TOP), ref_s, 1e-3,
                                  what=f"routed decode request {b}")
    # only the eight routed heads contribute: zeroing every other head's query leaves the logits unchanged
    qz = q_fp8.view(torch.uint8).clone().view(32, 64, 128)
    keep = torch.zeros(32, 64, dtype=torch.bool, device="cuda").scatter_(1, heads.long(), True)
    qz[~keep] = 0
    logits_z = K.indexer_paged_fp8_logits(qz.view(torch.float8_e4m3fn), gate.contiguous(), st.k_cache, 64,
                                          st.context_lens, st.block_table, max_cols=65536)
    assert torch.equal(logits_z, logits)
