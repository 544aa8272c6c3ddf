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
    # oracle spot check of the scores on three requests
    cache_cpu, table_cpu = st.k_cache.cpu(), st.block_table.cpu()
    keys = None
    for b in (3, 40):
        if keys is None:
            keys = O.unpack_paged_fp8_cache(cache_cpu, 64)
        kb = O.gather_request_keys(keys, table_cpu[b], lens[b])
        ref = O.indexer_scores(q_fp8[b:b + 1].cpu().float(), kb, wf[b:b + 1].cpu(), 1.0)[0]
        assert O.rel_err(logits[b, :lens[b]].cpu(), ref) < 1e-2          # stated FP8 tolerance


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
    # stage 2 is exact inside the kept blocks: compare with a dense scoring of those blocks by torch
    for t in (0, 100, 255):
        cols = (blocks[t].long().view(-1, 1) * 128 + torch.arange(128, device="cuda")).reshape(-1)
        sc = (torch.relu(q[t].float() @ k[cols].float().T) * w[t].view(-1, 1)).sum(0)
        sc[cols >= ke[t]] = float("-inf")
        ref = cols[torch.topk(sc, 2048).indices]
        assert len(set(ref.tolist()) & set(idx[t].tolist())) >= 2040


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
    # only the eight routed heads contribute: zeroing every other head's query leaves the logits unchanged
    qz = q_fp8.view(torch.uint8).clone().view(32, 64, 128)
    keep = torch.zeros(32, 64, dtype=torch.bool, device="cuda").scatter_(1, heads.long(), True)
    qz[~keep] = 0
    logits_z = K.indexer_paged_fp8_logits(qz.view(torch.float8_e4m3fn), gate.contiguous(), st.k_cache, 64,
                                          st.context_lens, st.block_table, max_cols=65536)
    assert torch.equal(logits_z, logits)
