"""The CPU oracle must reproduce what the reference's own OpenDSA ops returned on the
seeded inputs of tests/golden/make_golden.py (outputs stored as .npz)."""
import os

import numpy as np
import pytest
import torch

from oracle import dsa_oracle as O
from tests.golden.make_golden import (ATTEND_CASES, SELECT_CASES, golden_inputs_attend,
                                      golden_inputs_select)

GOLD = os.path.join(os.path.dirname(__file__), "golden")


@pytest.mark.parametrize("case", SELECT_CASES, ids=[c[0] for c in SELECT_CASES])
def test_select_matches_reference(case):
    name, seed, Lq, Lk, H, d, topk, docs, mode = case
    q, k, w, cu, gpos = golden_inputs_select(seed, Lq, Lk, H, d, docs, mode)
    g = np.load(os.path.join(GOLD, name + ".npz"))
    if gpos is None:
        ks, ke = O.prepare_ks_ke(cu)
    else:
        ks, ke = O.prepare_ks_ke_cp(cu, gpos)
    assert np.array_equal(ks.numpy(), g["ks"]) and np.array_equal(ke.numpy(), g["ke"])
    idx = O.indexer_select_topk(q, k, w, cu, topk, q_global_pos=gpos)
    ref = torch.from_numpy(g["idx"])
    # same arithmetic order as the reference on CPU -> identical rows, order included
    assert torch.equal(idx, ref)


@pytest.mark.parametrize("case", ATTEND_CASES, ids=[c[0] for c in ATTEND_CASES])
def test_attend_matches_reference(case):
    name, seed, L, H, Dl, d_c, K = case
    q, lat, W_UV, idx = golden_inputs_attend(seed, L, H, Dl, d_c, K)
    g = np.load(os.path.join(GOLD, name + ".npz"))
    ctx, lse = O.sparse_attend_latent(q, lat, idx, d_c=d_c, sm_scale=Dl ** -0.5)
    assert torch.allclose(ctx, torch.from_numpy(g["ctx"]), rtol=1e-5, atol=1e-6)
    out = O.sparse_attend_absorbed(q, lat, W_UV, idx, d_c=d_c, sm_scale=Dl ** -0.5)
    assert torch.allclose(out, torch.from_numpy(g["out"]), rtol=1e-5, atol=1e-6)
    assert torch.isinf(lse[3]).all() and (ctx[3] == 0).all()      # fully masked row


def test_lse_combine_equals_unsharded():
    g = torch.Generator().manual_seed(5)
    L, H, Dl, d_c, K = 6, 4, 24, 16, 40
    q = torch.randn(L, H, Dl, generator=g)
    lat = torch.randn(200, Dl, generator=g)
    idx = torch.randint(0, 200, (L, K), generator=g).to(torch.int32)
    qpos = torch.full((L,), 199)
    full, lse = O.sparse_attend_latent(q, lat, idx, d_c=d_c, sm_scale=0.2, q_pos=qpos)
    parts, lses = [], []
    for lo, hi in [(0, 50), (50, 100), (100, 200)]:
        own = torch.where((idx >= lo) & (idx < hi), idx, torch.full_like(idx, -1))
        c, l = O.sparse_attend_latent(q, lat, own, d_c=d_c, sm_scale=0.2, q_pos=qpos)
        parts.append(c); lses.append(l)
    out, lse2 = O.lse_combine(parts, lses)
    assert torch.allclose(out, full, rtol=1e-5, atol=1e-6)
    assert torch.allclose(lse2, lse, rtol=1e-5, atol=1e-6)


def test_paged_fp8_roundtrip_and_logits():
    g = torch.Generator().manual_seed(6)
    ctxs = [130, 64, 1, 257]
    P = 64
    ks = [torch.randn(c, 128, generator=g) for c in ctxs]
    qs = [O.quant_fp8_rows(k) for k in ks]
    cache, table = O.pack_paged_fp8_cache([a for a, _ in qs], [b for _, b in qs], P, 16, g)
    keys = O.unpack_paged_fp8_cache(cache, P)
    for b, c in enumerate(ctxs):
        kb = O.gather_request_keys(keys, table[b], c)
        assert torch.equal(kb, qs[b][0].float() * qs[b][1].unsqueeze(-1))
        assert (kb - ks[b]).abs().max() < 0.3
    q = torch.randn(len(ctxs), 64, 128, generator=g)
    w = torch.randn(len(ctxs), 64, generator=g) / 8
    lg = O.paged_indexer_logits(q, cache, w, torch.tensor(ctxs), table, P, 320, 128 ** -0.5)
    for b, c in enumerate(ctxs):
        assert torch.isinf(lg[b, c:]).all() and torch.isfinite(lg[b, :c]).all()


def test_hisa_equals_dense_when_all_blocks_kept():
    g = torch.Generator().manual_seed(7)
    T, S, H, d = 12, 300, 8, 32
    q = torch.randn(T, H, d, generator=g); k = torch.randn(S, d, generator=g)
    w = torch.randn(T, H, generator=g) / 8
    ke = torch.arange(S - T, S) + 1
    ks = torch.zeros(T, dtype=torch.int64)
    dense = O.topk_rows(O.mask_interval(O.indexer_scores(q, k, w), ks, ke), 32)
    hisa = O.hisa_select_topk(q, k, w, ks, ke, block=16, block_topk=19, topk=32)
    assert O.set_recall(hisa, dense) == 1.0


def test_block_mean_pool_tail():
    k = torch.arange(10, dtype=torch.float32).view(10, 1).repeat(1, 4)
    p = O.block_mean_pool(k, 4)
    assert torch.allclose(p[:, 0], torch.tensor([1.5, 5.5, 8.5]))


def test_indexer_producer_matches_reference_module():
    """The oracle's restatement of LightningIndexer.forward against the stored outputs of the
    reference module (tests/golden/make_golden.py, fp32)."""
    from tests.golden.make_golden import INDEXER_CASES, golden_inputs_indexer
    name, seed, B, L, hidden, H = INDEXER_CASES[0]
    h, cos, sin, state = golden_inputs_indexer(seed, B, L, hidden, H)
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", name + ".npz"))
    q, k, w = O.lightning_indexer_forward(h, h, cos, sin, state, H)
    for got, key in ((q, "q"), (k, "k"), (w, "w")):
        want = torch.from_numpy(g[key])
        assert got.shape == want.shape and (got - want).abs().max() < 1e-5 * want.abs().max().clamp_min(1.0)
