"""Drop-in OpenDSA ops and the HISA two-stage path against the oracle and the reference's
golden outputs."""
import os

import numpy as np
import pytest
import torch

from oracle import dsa_oracle as O
from tests.golden.make_golden import (ATTEND_CASES, SELECT_CASES, golden_inputs_attend, golden_inputs_select)

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")
BF16_RTOL = 2e-3


def _audit(idx, ref, scores, rtol=BF16_RTOL):
    rec = O.set_recall(idx, ref)
    total, bad = O.near_tie_audit(idx, ref, scores, rtol)
    return rec, total, bad


@pytest.mark.parametrize("case", [c for c in SELECT_CASES if c[4] in (64, 8, 4) and c[5] == 128],
                         ids=lambda c: c[0])
def test_select_golden_cases(case):
    from transarch_b200 import opendsa_ops as D
    name, seed, Lq, Lk, H, d, topk, docs, mode = case
    q, k, w, cu, gpos = golden_inputs_select(seed, Lq, Lk, H, d, docs, mode)
    g = np.load(os.path.join(GOLD, name + ".npz"))
    idx = D.indexer_select_topk(q.cuda(), k.cuda(), w.cuda(), cu.cuda(), topk,
                                q_global_pos=None if gpos is None else gpos.cuda()).cpu()
    # strict: oracle on the bf16-rounded operands the kernel sees
    qb, kb = q.bfloat16().float(), k.bfloat16().float()
    ks, ke = torch.from_numpy(g["ks"]), torch.from_numpy(g["ke"])
    scores = O.mask_interval(O.indexer_scores(qb, kb, w), ks, ke)
    ref_b = O.topk_rows(scores, topk)
    rec, total, bad = _audit(idx, ref_b, scores)
    assert rec >= 0.999 or bad == 0, (rec, total, bad)
    assert bad == 0
    # the reference's own fp32 output: same sets up to bf16 rounding of the operands
    assert O.set_recall(idx, torch.from_numpy(g["idx"])) >= 0.97
    # -1 padding exactly where the reference pads
    assert torch.equal(idx < 0, torch.from_numpy(g["idx"]) < 0)


def test_select_config1_shape_scores_and_sets():
    """Causal prefill T=S=4096, 64 heads, d=128, top-2048, seed 0 (the CPU-reference configuration)."""
    from transarch_b200 import opendsa_ops as D
    g = torch.Generator().manual_seed(0)
    T = 4096
    q = torch.randn(T, 64, 128, generator=g)
    k = torch.randn(T, 128, generator=g)
    w = torch.randn(T, 64, generator=g) / 8
    cu = torch.tensor([0, T])
    idx = D.indexer_select_topk(q.cuda(), k.cuda(), w.cuda(), cu.cuda(), 2048).cpu()
    qb, kb = q.bfloat16().float(), k.bfloat16().float()
    # index sets: ALL 4096 queries against the oracle (chunks keep the fp32 score matrix small)
    ksd, ked = D.prepare_ks_ke(cu.cuda())
    logits, _, _ = D.indexer_logits_flat(q.cuda().bfloat16(), k.cuda().bfloat16(), w.cuda(), ksd, ked, 128 ** -0.5)
    logits = logits.cpu()
    worst = 0.0
    for t0 in range(0, T, 512):
        t1 = t0 + 512
        ks, ke = torch.zeros(512, dtype=torch.int64), torch.arange(t0, t1) + 1
        scores = O.mask_interval(O.indexer_scores(qb[t0:t1], kb, w[t0:t1]), ks, ke)
        ref = O.topk_rows(scores, 2048)
        O.assert_selection_parity(idx[t0:t1], ref, scores, BF16_RTOL, what=f"queries {t0}..{t1}")
        assert torch.equal(idx[t0:t1] < 0, ref < 0)
        # scores themselves (bf16 tolerance)
        worst = max(worst, O.rel_err(logits[t0:t1, :T], scores))
    assert worst < BF16_RTOL, worst


def test_attend_golden_through_dropin():
    from transarch_b200 import opendsa_ops as D
    name, seed, L, H, Dl, d_c, Kk = ATTEND_CASES[1]
    q, lat, W_UV, idx = golden_inputs_attend(seed, L, H, Dl, d_c, Kk)
    g = np.load(os.path.join(GOLD, name + ".npz"))
    out = D.sparse_attend_absorbed_chunked(q.cuda(), lat.cuda(), W_UV.cuda(), idx.cuda(), d_c=d_c,
                                           sm_scale=Dl ** -0.5).cpu()
    ref = torch.from_numpy(g["out"])
    assert (out - ref).abs().max() / ref.abs().max() < 2e-2


def test_attend_gradients_match_reference_autograd():
    """Under autograd the drop-in is differentiable: d q_lat, d latent and d W_UV against autograd through
    the reference's own op (its files under oracle/_ref when present, else the oracle restatement) on the
    golden MLA-shaped case, which has -1 padding, future positions and an empty row.  2e-2 of the largest
    entry: the forward context is bf16."""
    from transarch_b200 import opendsa_ops as D
    from oracle import make_ref
    name, seed, L, H, Dl, d_c, Kk = ATTEND_CASES[1]
    q, lat, W_UV, idx = golden_inputs_attend(seed, L, H, Dl, d_c, Kk)
    q, lat = q.bfloat16().float(), lat.bfloat16().float()
    gen = torch.Generator().manual_seed(5)
    G = torch.randn(L, H, W_UV.shape[1], generator=gen)
    ref_ops = make_ref.reference_ops()

    def ref_fn(a, b, c):
        if ref_ops is not None:
            return ref_ops.sparse_attend_absorbed_chunked(a, b, c, idx, d_c=d_c, sm_scale=Dl ** -0.5, q_chunk=7)
        return O.sparse_attend_absorbed(a, b, c, idx, d_c=d_c, sm_scale=Dl ** -0.5)

    a, b, c = (t.clone().requires_grad_() for t in (q, lat, W_UV))
    (ref_fn(a, b, c) * G).sum().backward()
    x, y, z = (t.clone().cuda().requires_grad_() for t in (q, lat, W_UV))
    out = D.sparse_attend_absorbed_chunked(x, y, z, idx.cuda(), d_c=d_c, sm_scale=Dl ** -0.5, q_chunk=7)
    assert out.requires_grad
    (out * G.cuda()).sum().backward()
    for got, ref, what in ((x.grad, a.grad, "q_lat"), (y.grad, b.grad, "latent"), (z.grad, c.grad, "W_UV")):
        err = (got.cpu() - ref).abs().max() / ref.abs().max()
        assert err < 2e-2, (what, float(err))
    # bf16 inputs: the backward's products run in bf16 (fp32 accumulation); same gradients within bf16 accuracy
    xb, yb, zb = (t.clone().cuda().bfloat16().requires_grad_() for t in (q, lat, W_UV))
    outb = D.sparse_attend_absorbed_chunked(xb, yb, zb, idx.cuda(), d_c=d_c, sm_scale=Dl ** -0.5, q_chunk=7)
    (outb.float() * G.cuda()).sum().backward()
    for got, ref, what in ((xb.grad, a.grad, "q_lat"), (yb.grad, b.grad, "latent"), (zb.grad, c.grad, "W_UV")):
        assert got.dtype == torch.bfloat16
        err = (got.float().cpu() - ref).abs().max() / ref.abs().max()
        assert err < 4e-2, (what, float(err))
    # only some inputs need gradients
    x2 = q.clone().cuda().requires_grad_()
    out = D.sparse_attend_absorbed_chunked(x2, lat.cuda(), W_UV.cuda(), idx.cuda(), d_c=d_c, sm_scale=Dl ** -0.5)
    (out * G.cuda()).sum().backward()
    assert (x2.grad.cpu() - a.grad).abs().max() / a.grad.abs().max() < 2e-2


def test_hisa_two_stage_vs_oracle():
    from transarch_b200.hisa import HisaConfig, hisa_select_topk
    g = torch.Generator().manual_seed(2)
    T, S = 96, 16384 + 77
    q = torch.randn(T, 64, 128, generator=g).bfloat16()
    k = torch.randn(S, 128, generator=g).bfloat16()
    w = torch.randn(T, 64, generator=g) / 8
    ke = torch.arange(S - T, S) + 1
    ks = torch.zeros(T, dtype=torch.int64)
    ks[:8] = 3000                                              # a later document start
    cfg = HisaConfig(hisa_block_topk=16, index_topk=512)
    idx, blocks = hisa_select_topk(q.cuda(), k.cuda(), w.cuda(), ks.cuda(), ke.cuda(), cfg, return_blocks=True)
    idx, blocks = idx.cpu(), blocks.cpu()
    ref, ref_blocks = O.hisa_select_topk(q, k, w, ks, ke, block=128, block_topk=16, topk=512, return_blocks=True)
    # stage 1: the kept blocks, audited on the oracle's block scores (the forced block carries +inf)
    blk_scores = O.hisa_block_logits(q, O.block_mean_pool(k, 128), w, ks, ke, 128)
    blk_scores = O.finite_top(blk_scores)               # the forced block's +inf -> just above the row's best
    O.assert_selection_parity(blocks, ref_blocks, blk_scores, BF16_RTOL, what="HISA blocks")
    # stage 2: token picks inside the blocks the kernel itself kept
    ref2, tok_scores = O.hisa_select_topk(q, k, w, ks, ke, block=128, block_topk=16, topk=512, blocks=blocks,
                                          return_scores=True)
    O.assert_selection_parity(idx, ref2, tok_scores, BF16_RTOL, what="HISA tokens")
    # both stages end to end: a block-level near-tie moves up to 128 candidates at once
    assert O.set_recall(idx, ref) >= 0.999 or not torch.equal(torch.sort(blocks, 1).values,
                                                              torch.sort(ref_blocks, 1).values)
    last = ((ke + 127) // 128 - 1).to(torch.int32)
    assert (blocks[:, 0] == last).all()                   # the forced block sorts first (+inf)
    # quality: overlap with the dense selection (HISA's own claim is > 99 % IoU on real data;
    # on white-noise keys block means carry little signal, so only a sanity bound is asserted)
    dense = O.topk_rows(O.mask_interval(O.indexer_scores(q, k, w), ks, ke), 512)
    assert O.set_recall(idx, dense) > 0.1


def test_hisa_equals_dense_when_every_block_is_kept():
    from transarch_b200 import opendsa_ops as D
    from transarch_b200.hisa import HisaConfig, hisa_select_topk
    g = torch.Generator().manual_seed(3)
    T, S = 40, 128 * 9 + 5
    q = torch.randn(T, 64, 128, generator=g).bfloat16()
    k = torch.randn(S, 128, generator=g).bfloat16()
    w = torch.randn(T, 64, generator=g) / 8
    ke = (torch.arange(S - T, S) + 1).cuda()
    ks = torch.zeros(T, dtype=torch.int64).cuda()
    idx = hisa_select_topk(q.cuda(), k.cuda(), w.cuda(), ks, ke, HisaConfig(hisa_block_topk=10, index_topk=256))
    dense = D.indexer_select_topk(q.cuda(), k.cuda(), w.cuda(), torch.tensor([0, S]).cuda(), 256,
                                  q_global_pos=(ke - 1))
    assert torch.equal(torch.sort(idx, 1).values, torch.sort(dense, 1).values)


def test_hisa_paged_fp8_two_stage_vs_oracle():
    """HISA over the paged FP8 cache (decode rows, two rows per request): block selection and token
    selection against the oracle's two-stage restatement on the dequantised keys.  Power-of-two key scales
    make the dequantised keys exact in bf16, so both sides pool and score identical numbers."""
    from transarch_b200 import _lib, kernels as K
    from transarch_b200.hisa import HisaConfig, hisa_select_topk_paged
    P, ctxs, next_n = 64, [9000, 2500, 16384, 130], 2
    g = torch.Generator().manual_seed(21)
    qs = [O.quant_fp8_rows(torch.randn(c, 128, generator=g), ue8m0=True) for c in ctxs]
    n_pages = sum((c + P - 1) // P for c in ctxs) + 4
    cache, table = O.pack_paged_fp8_cache([a for a, _ in qs], [b for _, b in qs], P, n_pages, g)
    table = table.clamp(min=0)
    rows = len(ctxs) * next_n
    q = torch.randn(rows, 64, 128, generator=g)
    w = torch.randn(rows, 64, generator=g) / 8
    q_fp8, wf = O.quant_q_fold_weights(q, w, 128 ** -0.5, ue8m0=True)
    lens = torch.tensor(ctxs, dtype=torch.int32)
    row_ctx = (lens.view(-1, 1) - next_n + torch.arange(next_n, dtype=torch.int32).view(1, -1) + 1).reshape(-1)
    cfg = HisaConfig(hisa_block_topk=8, index_topk=256)
    idx, blocks = hisa_select_topk_paged(q_fp8.cuda(), wf.cuda(), cache.cuda(), P, row_ctx.cuda(), table.cuda(), cfg,
                                         next_n=next_n, return_blocks=True)
    assert _lib.read_status(idx.device) == 0
    idx, blocks = idx.cpu(), blocks.cpu()
    for r in range(rows):
        b, n = r // next_n, int(row_ctx[r])
        kd = (qs[b][0].float() * qs[b][1].unsqueeze(-1))[:n].bfloat16()
        ks, ke = torch.zeros(1, dtype=torch.int64), torch.tensor([n])
        qf, wr = q_fp8[r:r + 1].float(), wf[r:r + 1]
        blk_scores = O.finite_top(O.hisa_block_logits(qf, O.block_mean_pool(kd, 128), wr, ks, ke, 128, 1.0))
        ref_blocks = O.topk_rows(O.hisa_block_logits(qf, O.block_mean_pool(kd, 128), wr, ks, ke, 128, 1.0), 8,
                                 keep_pos_inf=True)
        O.assert_selection_parity(blocks[r:r + 1], ref_blocks, blk_scores, BF16_RTOL, what=f"row {r} blocks")
        ref2, tok_scores = O.hisa_select_topk(qf, kd, wr, ks, ke, block=128, block_topk=8, topk=256, sm_scale=1.0,
                                              blocks=blocks[r:r + 1], return_scores=True)
        O.assert_selection_parity(idx[r:r + 1], ref2, tok_scores, 1e-3, what=f"row {r} tokens")
        assert int(blocks[r, 0]) == (n + 127) // 128 - 1          # the row's last block is always kept


def test_patch_opendsa_rebinds_the_reference_names():
    """patch_opendsa() against the reference package itself (installed by oracle/make_ref.py): the names the
    reference's attention module bound at import now run this library, and its indexer module's state dict
    loads into ours unchanged."""
    import sys
    ref_dir = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref")
    if not os.path.exists(os.path.join(ref_dir, "opendsa", "modeling", "dsa_attention.py")):
        pytest.skip("oracle/_ref is not installed (python -m oracle.make_ref needs the TransArch checkout)")
    if ref_dir not in sys.path:
        sys.path.insert(0, ref_dir)
    import opendsa.modeling.dsa_attention as att
    import opendsa.ops as ops
    from opendsa.modeling.indexer import LightningIndexer as RefIndexer
    from transarch_b200 import opendsa_ops as D
    from transarch_b200.indexer_module import LightningIndexer
    ref_select, ref_attend = ops.indexer_select_topk, ops.sparse_attend_absorbed_chunked
    assert att.indexer_select_topk is ref_select
    try:
        D.patch_opendsa()
        assert att.indexer_select_topk is D.indexer_select_topk and ops.indexer_select_topk is D.indexer_select_topk
        assert att.sparse_attend_absorbed_chunked is D.sparse_attend_absorbed_chunked
        # through the patched module, on a golden case: the reference's own stored output
        name, seed, Lq, Lk, H, d, topk, docs, mode = [c for c in SELECT_CASES if c[0] == "select_packed_docs"][0]
        q, k, w, cu, gpos = golden_inputs_select(seed, Lq, Lk, H, d, docs, mode)
        g = np.load(os.path.join(GOLD, name + ".npz"))
        idx = att.indexer_select_topk(q.cuda(), k.cuda(), w.cuda(), cu.cuda(), topk).cpu()
        assert torch.equal(idx < 0, torch.from_numpy(g["idx"]) < 0)
        assert O.set_recall(idx, torch.from_numpy(g["idx"])) >= 0.97      # bf16 operands vs the fp32 reference run
    finally:
        for mod in (att, ops):
            mod.indexer_select_topk, mod.sparse_attend_absorbed_chunked = ref_select, ref_attend
    # the indexer module: same parameter names and shapes, and the same outputs on the reference's CPU run
    ref_mod = RefIndexer(48, n_heads=8, dtype=torch.float32)
    mine = LightningIndexer(48, n_heads=8, dtype=torch.float32)
    mine.load_state_dict(ref_mod.state_dict(), strict=True)
    g2 = torch.Generator().manual_seed(5)
    h = torch.randn(1, 9, 48, generator=g2)
    ang = torch.rand(1, 9, 32, generator=g2) * 6.28
    cos, sin = torch.cat([ang.cos(), ang.cos()], -1), torch.cat([ang.sin(), ang.sin()], -1)
    with torch.no_grad():
        rq, rk, rw = ref_mod(h, h, cos, sin)
    torch.backends.cuda.matmul.allow_tf32 = False
    mq, mk, mw = mine.cuda()(h.cuda(), h.cuda(), cos.cuda(), sin.cuda())
    for a, b in ((mq, rq), (mk, rk), (mw, rw)):
        assert (a.cpu() - b).abs().max() < 2e-4 * b.abs().max()


def test_causal_row_intervals_equal_the_torch_helpers():
    """One launch gives what prepare_ks_ke / prepare_ks_ke_cp and the column-frame arithmetic give."""
    from transarch_b200 import kernels as K
    from transarch_b200.opendsa_ops import prepare_ks_ke, prepare_ks_ke_cp
    cu = torch.tensor([0, 5, 5, 700, 701, 4096], dtype=torch.int32, device="cuda")      # an empty document too
    lo, hi, col0, rc = K.causal_row_intervals(cu, 4096)
    ks, ke = prepare_ks_ke(cu, total=4096)
    assert torch.equal(lo.long(), ks) and torch.equal(hi.long(), ke)
    assert torch.equal(col0, (lo >> 7) << 7)
    assert torch.equal(rc, ((((hi + 127) >> 7) << 7) - col0).clamp(min=0))
    g = torch.Generator().manual_seed(1)
    pos = torch.randint(0, 4096, (333,), generator=g).cuda()
    lo, hi, col0, rc = K.causal_row_intervals(cu, 333, pos)
    ks, ke = prepare_ks_ke_cp(cu, pos)
    assert torch.equal(lo.long(), ks) and torch.equal(hi.long(), ke)
    assert torch.equal(rc, ((((hi + 127) >> 7) << 7) - ((lo >> 7) << 7)).clamp(min=0))
