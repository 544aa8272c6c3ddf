"""The reference's own TileLang kernels, JIT-compiled on this GPU, as a comparator for the MISA path.

oracle/make_ref.py installs the two kernel files of the reference (misa_ops.py, block_ops.py: torch +
tilelang only) into the git-ignored oracle/_ref/.  Where TileLang lowers a kernel for this GPU the
reference's function is run on the same seeded inputs as this library's; where it does not, the case is
skipped with TileLang's error.  Inputs are chosen so that both sides see the same numbers: head weights
already rounded to bf16 (the reference rounds them, misa_ops.py:690 / :376) and power-of-two key scales
(fp8 * 2^e is exact in bf16, so the reference's whole-cache dequantisation to bf16 loses nothing)."""
import os
import sys

import pytest
import torch

from oracle import dsa_oracle as O

pytestmark = pytest.mark.gpu

REF_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref")
BF16_RTOL = 2e-3


def _ref_modules():
    if not os.path.exists(os.path.join(REF_DIR, "misa_vllm_patch", "misa_ops.py")):
        pytest.skip("oracle/_ref is not installed (python -m oracle.make_ref needs the TransArch checkout)")
    pytest.importorskip("tilelang")
    if REF_DIR not in sys.path:
        sys.path.insert(0, REF_DIR)
    from misa_vllm_patch import block_ops, misa_ops
    return misa_ops, block_ops


def _run_ref(fn, *a, **k):
    try:
        return fn(*a, **k)
    except Exception as e:  # noqa: BLE001 - a TileLang lowering / compile failure closes the case
        pytest.skip(f"TileLang could not run {getattr(fn, '__name__', fn)} here: {type(e).__name__}: {str(e)[-300:]}")


def _common_logit_err(logits, cand, ref_logits, ref_cand, n_cols):
    """Largest difference of the stage-2 logits on candidates both sides shortlisted, relative to rms."""
    M = cand.shape[0]
    a = torch.full((M, n_cols), float("nan"))
    b = torch.full((M, n_cols), float("nan"))
    ok = cand >= 0
    a[torch.arange(M).view(-1, 1).expand_as(cand)[ok], cand[ok].long()] = logits[ok]
    okr = ref_cand >= 0
    b[torch.arange(M).view(-1, 1).expand_as(ref_cand)[okr], ref_cand[okr].long()] = ref_logits[okr]
    both = torch.isfinite(a) & torch.isfinite(b)
    assert int(both.sum()) > 0.9 * int(ok.sum())
    return float((a[both] - b[both]).abs().max() / a[both].pow(2).mean().sqrt())


def test_block_mean_pooling_bitwise():
    _, RB = _ref_modules()
    from transarch_b200 import kernels as K
    g = torch.Generator().manual_seed(42)
    for n in (4096, 1000, 129):
        k = torch.randn(n, 128, generator=g).bfloat16().cuda()
        ref = _run_ref(RB.block_mean_pooling_interface, k, 128)
        assert torch.equal(K.block_mean_pool(k, 128), ref.to(torch.bfloat16))


@pytest.mark.parametrize("use_qnorm", [True, False])
def test_flat_two_stage_logits_against_tilelang(use_qnorm):
    """misa_mqa_logits (misa_ops.py:653-713): head routing, stage-1 shortlist, all-head re-score."""
    RM, _ = _ref_modules()
    from transarch_b200 import misa as M
    g = torch.Generator().manual_seed(43)
    Mq, N, s1 = 256, 4096, 1024
    kq, sc = O.quant_fp8_rows(torch.randn(N, 128, generator=g), ue8m0=True)
    q = torch.randn(Mq, 64, 128, generator=g)
    w = torch.randn(Mq, 64, generator=g) / 8
    q_fp8, wf = O.quant_q_fold_weights(q, w, 128 ** -0.5, 64 ** -0.5, ue8m0=True)
    wf = wf.bfloat16().float()                                       # what the reference's kernels see
    ke = torch.arange(N - Mq, N, dtype=torch.int32) + 1
    ks = torch.zeros(Mq, dtype=torch.int32)
    ks[:16] = 1000                                                    # a later document start
    hidx = O.qnorm_head_topk(q, 8) if use_qnorm else None
    args = (q_fp8.cuda(), (kq.cuda(), sc.cuda()), wf.cuda(), None if hidx is None else hidx.cuda(), ks.cuda(),
            ke.cuda(), use_qnorm, 8, s1)
    ref_logits, ref_cand = _run_ref(RM.misa_mqa_logits, *args, k_block_size=128)
    logits, cand = M.misa_mqa_logits(*args, k_block_size=128)
    ref_cand, cand = ref_cand.cpu().to(torch.int32), cand.cpu()
    # the reference's torch.topk also returns masked (-inf) columns for rows with fewer than s1 keys
    ref_valid = torch.isfinite(ref_logits.cpu())
    ref_cand = torch.where(ref_valid, ref_cand, torch.full_like(ref_cand, -1))
    kb = kq.float() * sc.unsqueeze(-1)
    qf = q_fp8.float()
    if hidx is None:          # the heads the block-score router keeps, from the oracle (audited through stage 1)
        pooled = O.block_mean_pool(kb.bfloat16(), 128).float()
        hidx = torch.topk(O.misa_block_head_scores(qf, pooled, wf, ks.long() // 128, (ke.long() + 127) // 128), 8).indices
    q8, w8 = O.gather_heads(qf, wf, hidx)
    st1 = O.mask_interval(O.indexer_scores(q8, kb, w8, 1.0), ks.long(), ke.long())
    O.assert_selection_parity(cand, ref_cand, st1, BF16_RTOL, what="stage-1 shortlist vs the reference's TileLang kernels")
    assert _common_logit_err(logits.cpu(), cand, ref_logits.cpu().float(), ref_cand, N) < BF16_RTOL


@pytest.mark.parametrize("use_qnorm", [True, False])
def test_paged_two_stage_logits_against_tilelang(use_qnorm):
    """misa_page_mqa_logits (misa_ops.py:344-413) over a paged FP8 cache with a shuffled block table."""
    RM, _ = _ref_modules()
    from transarch_b200 import misa as M
    P, ctxs, max_len, s1 = 64, [3000, 700, 4096, 1500], 4096, 512
    g = torch.Generator().manual_seed(44)
    qs = [O.quant_fp8_rows(torch.randn(c, 128, generator=g), ue8m0=True) for c in ctxs]
    n_pages = sum((c + P - 1) // P for c in ctxs) + 5
    cache, table = O.pack_paged_fp8_cache([a for a, _ in qs], [b for _, b in qs], P, n_pages, g)
    table = table.clamp(min=0)
    B = len(ctxs)
    q = torch.randn(B, 64, 128, generator=g)
    w = torch.randn(B, 64, generator=g) / 8
    q_fp8, wf = O.quant_q_fold_weights(q, w, 128 ** -0.5, 64 ** -0.5, ue8m0=True)
    wf = wf.bfloat16().float()
    lens = torch.tensor(ctxs, dtype=torch.int32)
    hidx = O.qnorm_head_topk(q, 8) if use_qnorm else None
    cache4 = cache.view(n_pages, P, 1, 132).cuda()
    args = (q_fp8.view(B, 1, 64, 128).cuda(), cache4, wf.cuda(), None if hidx is None else hidx.cuda(), lens.cuda(),
            table.cuda(), max_len, 8, use_qnorm, s1)
    ref_logits, ref_cand = _run_ref(RM.misa_page_mqa_logits, *args, k_block_size=128)
    logits, cand = M.misa_page_mqa_logits(*args, k_block_size=128)
    ref_logits, ref_cand, logits, cand = ref_logits.cpu().float(), ref_cand.cpu().to(torch.int32), logits.cpu(), cand.cpu()
    ref_cand = torch.where(torch.isfinite(ref_logits), ref_cand, torch.full_like(ref_cand, -1))
    st1 = torch.full((B, max_len), float("-inf"))
    for b, c in enumerate(ctxs):
        kd = qs[b][0].float() * qs[b][1].unsqueeze(-1)
        h = hidx[b:b + 1] if hidx is not None else torch.topk(O.misa_block_head_scores(
            q_fp8[b:b + 1].float(), O.block_mean_pool(kd, 128), wf[b:b + 1], torch.zeros(1, dtype=torch.long),
            torch.tensor([(c + 127) // 128])), 8).indices
        q8, w8 = O.gather_heads(q_fp8[b:b + 1].float(), wf[b:b + 1], h)
        st1[b, :c] = O.indexer_scores(q8, kd, w8, 1.0)[0]
    O.assert_selection_parity(cand, ref_cand, st1, BF16_RTOL, what="paged stage-1 shortlist vs TileLang")
    assert _common_logit_err(logits, cand, ref_logits, ref_cand, max_len) < BF16_RTOL


def test_clean_and_force_keep_masks_against_tilelang():
    """clean_and_maintain_logits_ (block_ops.py:636-666): -inf outside [ks, ke), +inf at ks and ke-1; the
    HISA stage-1 block scores with both ends force-kept must carry the same mask."""
    _, RB = _ref_modules()
    from transarch_b200 import kernels as K
    from transarch_b200.hisa import HisaConfig, hisa_block_logits
    g = torch.Generator().manual_seed(45)
    T, S = 64, 128 * 4096 - 100      # 4096 key blocks: the row length the reference kernel tiles by (block_K = 4096)
    q = torch.randn(T, 64, 128, generator=g).bfloat16().cuda()
    w = (torch.randn(T, 64, generator=g) / 8).cuda()
    k = torch.randn(S, 128, generator=g).bfloat16().cuda()
    ke = (torch.arange(S - T, S) + 1).cuda()
    ks = torch.zeros(T, dtype=torch.int64).cuda()
    ks[:8] = 3000
    pooled = K.block_mean_pool(k, 128)
    cfg = HisaConfig(keep_first_block=True, keep_last_block=True)
    mine = hisa_block_logits(q, pooled, w, ks, ke, cfg, 128 ** -0.5)
    wide = hisa_block_logits(q, pooled, w, torch.zeros_like(ks), torch.full_like(ke, S),
                             HisaConfig(keep_first_block=False, keep_last_block=False), 128 ** -0.5)
    bks = (ks // 128).to(torch.int32).contiguous()
    bke = ((ke + 127) // 128).to(torch.int32).contiguous()
    ref = wide.clone()
    kern = _run_ref(RB.clean_and_maintain_logits_)
    _run_ref(kern, ref, bks, bke)
    assert mine.shape[1] == 4096 and pooled.shape[0] == 4096
    assert torch.equal(mine, ref)


def test_paged_block_sparse_logits_against_tilelang():
    """paged_block_sparse_mqa_attn_return_logits (block_ops.py:151-379): token logits inside listed
    128-key blocks of the paged cache."""
    _, RB = _ref_modules()
    from transarch_b200 import kernels as K
    P, ctxs, m = 64, [3000, 700, 4096], 8
    g = torch.Generator().manual_seed(46)
    qs = [O.quant_fp8_rows(torch.randn(c, 128, generator=g), ue8m0=True) for c in ctxs]
    n_pages = sum((c + P - 1) // P for c in ctxs) + 5
    cache, table = O.pack_paged_fp8_cache([a for a, _ in qs], [b for _, b in qs], P, n_pages, g)
    table = table.clamp(min=0)
    B = len(ctxs)
    q = torch.randn(B, 64, 128, generator=g)
    w = torch.randn(B, 64, generator=g) / 8
    q_fp8, wf = O.quant_q_fold_weights(q, w, 128 ** -0.5, 64 ** -0.5, ue8m0=True)
    wf = wf.bfloat16().float()
    lens = torch.tensor(ctxs, dtype=torch.int32)
    blocks = torch.stack([torch.randperm((c + 127) // 128, generator=g)[:m] if (c + 127) // 128 >= m else
                          torch.cat([torch.randperm((c + 127) // 128, generator=g),
                                     torch.full((m - (c + 127) // 128,), 0, dtype=torch.long)]) for c in ctxs]).to(torch.int32)
    keys_bf16 = O.unpack_paged_fp8_cache(cache, P).bfloat16().view(n_pages, P, 1, 128).cuda()
    ref = _run_ref(RB.paged_block_sparse_mqa_attn_return_logits_interface, q_fp8.bfloat16().view(B, 1, 64, 128).cuda(),
                   keys_bf16, blocks.view(B, 1, m).cuda(), 128, wf.bfloat16().cuda(), lens.cuda(), table.cuda())
    row_cols = torch.full((B,), m * 128, dtype=torch.int32)
    mine = K.indexer_paged_blocklist_fp8_logits(q_fp8.cuda(), wf.cuda(), cache.cuda(), P, lens.cuda(), table.cuda(),
                                                blocks.cuda(), row_cols.cuda())
    ref = ref.float().view(B, m * 128).cpu()
    mine = mine.cpu()
    assert torch.equal(torch.isinf(ref), torch.isinf(mine))
    fin = torch.isfinite(ref)
    assert float((ref[fin] - mine[fin]).abs().max() / mine[fin].pow(2).mean().sqrt()) < BF16_RTOL
