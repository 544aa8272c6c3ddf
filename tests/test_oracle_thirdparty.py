"""The oracle's restatements of third-party arithmetic (not under the TransArch checkout) against an
independent implementation that is installed here: vLLM's pure-torch fp8_paged_mqa_logits_torch /
fp8_mqa_logits_torch (the functions the reference's indexers.py falls back to when DeepGEMM is absent,
indexers.py:109-132, :193-201 in its pinned vLLM).  This pins the paged FP8 cache layout (page =
page_size*128 e4m3 bytes, then page_size fp32 scales), the score formula on quantised operands and the
-inf fill beyond each context.  Only the single-token branch of the paged function is used: its
multi-token branch reads every token as 128 value bytes followed by its own 4 scale bytes, which
contradicts both its single-token branch and the reader in the reference (misa_ops.py:360-372).
CPU only."""
import pytest
import torch

from oracle import dsa_oracle as O

vllm_ops = pytest.importorskip("vllm.v1.attention.ops.rocm_aiter_mla_sparse")


def _cache(seed, ctxs, P=64):
    g = torch.Generator().manual_seed(seed)
    qs = [O.quant_fp8_rows(torch.randn(c, 128, generator=g), ue8m0=(seed % 2 == 0)) for c in ctxs]
    n_pages = sum((c + P - 1) // P for c in ctxs) + 3
    cache, table = O.pack_paged_fp8_cache([a for a, _ in qs], [b for _, b in qs], P, n_pages, g)
    return g, qs, cache, table.clamp(min=0)


def test_paged_layout_and_scores_match_vllm_torch_single_token():
    ctxs, P, max_len = [300, 64, 1000, 129], 64, 1024
    g, qs, cache, table = _cache(70, ctxs, P)
    B = len(ctxs)
    q = torch.randn(B, 64, 128, generator=g)
    w = torch.randn(B, 64, generator=g) / 8
    q_fp8, wf = O.quant_q_fold_weights(q, w, 128 ** -0.5, 64 ** -0.5, ue8m0=True)
    lens = torch.tensor(ctxs, dtype=torch.int32)
    ours = O.paged_indexer_logits(q_fp8.float(), cache, wf, lens, table, P, max_len)
    theirs = vllm_ops.fp8_paged_mqa_logits_torch(q_fp8.view(B, 1, 64, 128), cache.view(-1, P, 1, 132), wf, lens,
                                                 table, max_len)
    assert torch.equal(torch.isinf(ours), torch.isinf(theirs))
    assert O.rel_err(ours, theirs) < 1e-4        # fp32 summation order only


def test_flat_scores_match_vllm_torch():
    g = torch.Generator().manual_seed(72)
    M, N = 16, 700
    kq, sc = O.quant_fp8_rows(torch.randn(N, 128, generator=g))
    q_fp8, wf = O.quant_q_fold_weights(torch.randn(M, 64, 128, generator=g), torch.randn(M, 64, generator=g) / 8,
                                       128 ** -0.5, 64 ** -0.5)
    ks = torch.zeros(M, dtype=torch.int32)
    ke = torch.arange(N - M, N, dtype=torch.int32) + 1
    theirs = vllm_ops.fp8_mqa_logits_torch(q_fp8, (kq, sc), wf, ks, ke)
    ours = O.mask_interval(O.indexer_scores(q_fp8.float(), kq.float() * sc.unsqueeze(-1), wf, 1.0), ks.long(), ke.long())
    assert torch.equal(torch.isinf(ours), torch.isinf(theirs))
    # theirs rounds every per-head product sum to bf16 before the head reduction: compare against the
    # spread of the scores, not element-wise relative
    fin = torch.isfinite(ours)
    err = (ours[fin] - theirs[fin]).abs().max() / ours[fin].pow(2).mean().sqrt()
    assert err < 2e-2, err


def test_ue8m0_scale_is_the_published_formula():
    """exp2(ceil(log2(max(amax, eps) / 448))), evaluated exactly."""
    g = torch.Generator().manual_seed(73)
    x = torch.randn(5000, 128, generator=g) * torch.rand(5000, 1, generator=g) * 8
    x[0] = 0
    x[1] = 448.0 / 256                                    # amax/448 an exact power of two stays put
    for eps in (1e-4, 1e-10):
        q, s = O.quant_fp8_rows(x, ue8m0=True, eps=eps)
        raw = x.abs().amax(-1).clamp_min(eps) / 448.0
        want = torch.exp2(torch.ceil(torch.log2(raw.double()))).float()
        assert torch.equal(s, want)
        assert (s >= raw).all() and (s < 2 * raw).all()
        assert float(s[1]) == 2.0 ** -8
        deq = q.float() * s.unsqueeze(-1)
        assert ((deq - x).abs() <= s.unsqueeze(-1) * 16 + 1e-30).all()      # e4m3 step at the top binade is 32*scale
    q0, s0 = O.quant_fp8_rows(x, ue8m0=False)
    assert torch.equal(s0, x.abs().amax(-1).clamp_min(1e-4) / 448.0)
