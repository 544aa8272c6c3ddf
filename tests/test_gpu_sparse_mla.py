"""tcgen05 sparse MLA decode kernel against the oracle (and, through it, the reference's
sparse_attend_absorbed_chunked golden outputs)."""
import os

import numpy as np
import pytest
import torch

from oracle import dsa_oracle as O
from tests.golden.make_golden import ATTEND_CASES, golden_inputs_attend

pytestmark = pytest.mark.gpu

ATTN_RTOL = 2e-2   # stated tolerance for bf16 attention output
GOLD = os.path.join(os.path.dirname(__file__), "golden")


def _check(ctx, lse, ref_ctx, ref_lse):
    assert torch.isfinite(ctx).all()
    err = (ctx - ref_ctx).abs().max() / ref_ctx.abs().max().clamp_min(1e-6)
    assert err < ATTN_RTOL, f"ctx err {err}"
    fin = torch.isfinite(ref_lse)
    assert torch.equal(torch.isfinite(lse), fin)
    assert (lse[fin] - ref_lse[fin]).abs().max() < 2e-2


def test_golden_mla_shape_matches_reference_output():
    """Same seeded inputs as the stored reference run (rounded to bf16 for the kernel)."""
    from transarch_b200 import _lib, kernels as K
    name, seed, L, H, Dl, d_c, Kk = ATTEND_CASES[1]
    q, lat, W_UV, idx = golden_inputs_attend(seed, L, H, Dl, d_c, Kk)
    g = np.load(os.path.join(GOLD, name + ".npz"))
    qpos = torch.arange(L, dtype=torch.int32)
    ctx, lse = K.sparse_mla_decode(q.bfloat16().cuda(), lat.bfloat16().cuda(), idx.cuda(), Dl ** -0.5,
                                   q_pos=qpos.cuda())
    assert _lib.read_status(ctx.device) == 0
    ref = torch.from_numpy(g["ctx"])
    err = (ctx.cpu() - ref).abs().max() / ref.abs().max()
    assert err < ATTN_RTOL
    assert (ctx.cpu()[3] == 0).all() and torch.isinf(lse.cpu()[3]).all()    # fully masked row


@pytest.mark.parametrize("n_items,H,n_idx,ctx_len", [(3, 128, 2048, 5000), (2, 16, 64, 300), (4, 128, 100, 4000),
                                                      (1, 128, 33, 50)])
@pytest.mark.parametrize("pair", [False, True], ids=["heads_split", "cluster_pair"])
def test_decode_vs_oracle(n_items, H, n_idx, ctx_len, pair):
    from transarch_b200 import _lib, kernels as K
    g = torch.Generator().manual_seed(n_idx + H)
    q = torch.randn(n_items, H, 576, generator=g).bfloat16()
    kv = (0.5 * torch.randn(n_items * ctx_len, 576, generator=g)).bfloat16()
    base = torch.arange(n_items, dtype=torch.int64) * ctx_len
    idx = torch.stack([torch.randperm(ctx_len, generator=g)[:n_idx] for _ in range(n_items)]).to(torch.int32)
    idx[:, ::7] = -1
    qpos = torch.full((n_items,), ctx_len - 1, dtype=torch.int32)
    qpos[0] = ctx_len // 2                                  # masks about half of item 0's picks
    scale = 192 ** -0.5
    ctx, lse = K.sparse_mla_decode(q.cuda(), kv.cuda(), idx.cuda(), scale, kv_row_base=base.cuda(),
                                   q_pos=qpos.cuda(), pair=pair)
    assert _lib.read_status(ctx.device) == 0
    for b in range(n_items):
        rc, rl = O.sparse_attend_latent(q[b:b + 1], kv[b * ctx_len:(b + 1) * ctx_len], idx[b:b + 1],
                                        d_c=512, sm_scale=scale, q_pos=qpos[b:b + 1])
        _check(ctx[b:b + 1].cpu(), lse[b:b + 1].cpu(), rc, rl)
    # bf16 result buffer (the dtype the reference op returns): the fp32 result rounded once
    out16 = torch.empty(n_items, H, 512, dtype=torch.bfloat16, device="cuda")
    ctx16, lse16 = K.sparse_mla_decode(q.cuda(), kv.cuda(), idx.cuda(), scale, kv_row_base=base.cuda(),
                                       q_pos=qpos.cuda(), ctx=out16, pair=pair)
    assert ctx16.dtype == torch.bfloat16 and torch.equal(ctx16, ctx.bfloat16()) and torch.equal(lse16, lse)


@pytest.mark.parametrize("pair", [False, True], ids=["heads_split", "cluster_pair"])
def test_shard_partials_merge_to_full(pair):
    """Two position shards attended separately and merged by log-sum-exp equal the full result."""
    from transarch_b200 import kernels as K
    g = torch.Generator().manual_seed(77)
    n, H, n_idx, ctx_len = 2, 128, 512, 3000
    q = torch.randn(n, H, 576, generator=g).bfloat16()
    kv = (0.5 * torch.randn(ctx_len, 576, generator=g)).bfloat16()
    idx = torch.stack([torch.randperm(ctx_len, generator=g)[:n_idx] for _ in range(n)]).to(torch.int32)
    scale = 192 ** -0.5
    full_ctx, full_lse = O.sparse_attend_latent(q, kv, idx, d_c=512, sm_scale=scale,
                                                q_pos=torch.full((n,), ctx_len - 1))
    parts, lses = [], []
    for lo, hi in [(0, 1400), (1400, ctx_len)]:
        c, l = K.sparse_mla_decode(q.cuda(), kv[lo:hi].contiguous().cuda(), idx.cuda(), scale,
                                   pos_lo=lo, pos_hi=hi, pair=pair)
        parts.append(c.cpu()); lses.append(l.cpu())
    out, lse = O.lse_combine(parts, lses)
    _check(out, lse, full_ctx, full_lse)


@pytest.mark.parametrize("pair", [False, True], ids=["heads_split", "cluster_pair"])
def test_large_scores_trigger_rescale(pair):
    """Keys ordered so that the running maximum keeps growing: exercises the O rescale path (in the
    cluster-of-two kernel also the factors that travel to the partner CTA)."""
    from transarch_b200 import kernels as K
    g = torch.Generator().manual_seed(78)
    H, n_idx = 128, 256
    q = torch.randn(1, H, 576, generator=g).bfloat16()
    kv = torch.randn(n_idx, 576, generator=g)
    kv = (kv * torch.linspace(0.2, 6.0, n_idx).view(-1, 1)).bfloat16()   # later keys: far larger scores
    idx = torch.arange(n_idx, dtype=torch.int32).view(1, -1)
    scale = 0.3
    ctx, lse = K.sparse_mla_decode(q.cuda(), kv.cuda(), idx.cuda(), scale, pair=pair)
    rc, rl = O.sparse_attend_latent(q, kv, idx, d_c=512, sm_scale=scale, q_pos=torch.tensor([n_idx]))
    _check(ctx.cpu(), lse.cpu(), rc, rl)


@pytest.mark.parametrize("pair", [False, True], ids=["heads_split", "cluster_pair"])
def test_out_of_range_row_is_skipped_and_reported(pair):
    """An index that points past the latent cache is not read: the kernel drops that key, raises the
    status word to 2 (a skipped index) and the result equals attention over the remaining keys."""
    from transarch_b200 import _lib, kernels as K
    g = torch.Generator().manual_seed(9)
    n_items, H, n_idx, rows = 2, 128, 200, 1000
    q = torch.randn(n_items, H, 576, generator=g).bfloat16()
    kv = (0.5 * torch.randn(rows, 576, generator=g)).bfloat16()
    idx = torch.stack([torch.randperm(rows, generator=g)[:n_idx] for _ in range(n_items)]).to(torch.int32)
    bad = idx.clone()
    bad[1, 17] = rows + 5                                        # one row beyond the cache
    scale = 192 ** -0.5
    dev = torch.device("cuda")
    assert _lib.read_status(dev) == 0
    ctx, lse = K.sparse_mla_decode(q.cuda(), kv.cuda(), bad.cuda(), scale, pair=pair)
    torch.cuda.synchronize()
    assert _lib.read_status(dev) == 2
    good = idx.clone()
    good[1, 17] = -1
    for b in range(n_items):
        rc, rl = O.sparse_attend_latent(q[b:b + 1], kv, good[b:b + 1], d_c=512, sm_scale=scale,
                                        q_pos=torch.tensor([rows]))
        _check(ctx[b:b + 1].cpu(), lse[b:b + 1].cpu(), rc, rl)
    # the word was cleared by the read; a clean call leaves it at 0
    K.sparse_mla_decode(q.cuda(), kv.cuda(), good.cuda(), scale, pair=pair)
    torch.cuda.synchronize()
    assert _lib.read_status(dev) == 0


def test_cluster_pair_kernel_agrees_with_heads_split_kernel():
    """Same inputs through both attention kernels (64 items, 96 heads: the pair kernel pads to 128 rows)."""
    from transarch_b200 import _lib, kernels as K
    g = torch.Generator().manual_seed(31)
    n, H, n_idx, rows = 64, 96, 700, 20000
    q = torch.randn(n, H, 576, generator=g).bfloat16().cuda()
    kv = (0.5 * torch.randn(rows, 576, generator=g)).bfloat16().cuda()
    idx = torch.randint(0, rows, (n, n_idx), generator=g).to(torch.int32).cuda()
    idx[:, 5::11] = -1
    lens = torch.randint(0, n_idx + 1, (n,), generator=g).to(torch.int32).cuda()
    lens[0] = 0                                                     # an item without keys
    a, la = K.sparse_mla_decode(q, kv, idx, 0.07, n_idx_item=lens)
    b, lb = K.sparse_mla_decode(q, kv, idx, 0.07, n_idx_item=lens, pair=True)
    assert _lib.read_status(q.device) == 0
    assert (a[0] == 0).all() and (b[0] == 0).all() and torch.isinf(lb[0]).all()
    assert torch.equal(torch.isfinite(la), torch.isfinite(lb))
    fin = torch.isfinite(la)
    assert (la[fin] - lb[fin]).abs().max() < 1e-3
    assert (a - b).abs().max() / a.abs().max() < 5e-3


@pytest.mark.parametrize("T,H,dv", [(64, 128, 128), (200, 16, 96), (5, 8, 8), (129, 3, 256)])
def test_wuv_up_projection_matches_einsum(T, H, dv):
    """out[t,h,:] = ctx[t,h,:] @ W_UV[h]^T (OpenDSA/opendsa/ops/sparse_mla.py:44) on tensor cores."""
    from transarch_b200 import _lib, kernels as K
    g = torch.Generator().manual_seed(T + dv)
    ctx = torch.randn(T, H, 512, generator=g).bfloat16()
    w = (torch.randn(H, dv, 512, generator=g) / 512 ** 0.5).bfloat16()
    ref = torch.einsum("thl,hvl->thv", ctx.float(), w.float())
    out32 = K.wuv_up_project(ctx.cuda(), w.cuda(), out_dtype=torch.float32)
    out16 = K.wuv_up_project(ctx.cuda(), w.cuda())
    assert _lib.read_status(out32.device) == 0
    assert (out32.cpu() - ref).abs().max() < 1e-4 * ref.abs().max()        # bf16 products are exact in fp32
    assert (out16.float().cpu() - ref).abs().max() < 1e-2 * ref.abs().max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_backward_support_kernels(dtype):
    """The two kernels of the attention backward against the same arithmetic in framework operations:
    p / ds from raw scores (padding, future positions, a query without keys), and the fp32 scatter-add of the
    per-(query, key) row gradients into d_latent (duplicates, skipped entries, an index beyond the rows)."""
    from transarch_b200 import _lib, kernels as K
    g = torch.Generator().manual_seed(9)
    T, H, Kk, N = 13, 5, 40, 50
    s = torch.randn(T, H, Kk, generator=g).to(dtype)
    dp = torch.randn(T, H, Kk, generator=g).to(dtype)
    idx = torch.randint(0, N, (T, Kk), generator=g, dtype=torch.int32)
    idx[torch.rand(T, Kk, generator=g) < 0.2] = -1
    q_pos = torch.randint(10, N, (T,), generator=g, dtype=torch.int32)
    lse = torch.randn(T, H, generator=g) + 2.0
    lse[3] = float("-inf")                                    # a query that saw no key
    delta = torch.randn(T, H, generator=g)
    scale = 0.37
    p, ds = K.sparse_attn_bwd_pointwise(s.cuda(), dp.cuda(), lse.cuda(), delta.cuda(), idx.cuda(), q_pos.cuda(), scale)
    valid = ((idx >= 0) & (idx <= q_pos.view(-1, 1))).unsqueeze(1) & torch.isfinite(lse).unsqueeze(-1)
    p_ref = torch.where(valid, torch.exp(s.float() * scale - lse.unsqueeze(-1)), torch.zeros(T, H, Kk))
    ds_ref = p_ref * (dp.float() - delta.unsqueeze(-1)) * scale
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert p.dtype == dtype and torch.allclose(p.float().cpu(), p_ref, rtol=tol, atol=tol)
    assert torch.allclose(ds.float().cpu(), ds_ref, rtol=tol, atol=tol)
    # scatter-add
    a = torch.randn(T, Kk, 576, generator=g).to(dtype)
    b = torch.randn(T, Kk, 512, generator=g).to(dtype)
    d_lat = torch.zeros(N, 576, device="cuda")
    K.scatter_add_latent_rows(d_lat, a.cuda(), b.cuda(), idx.cuda(), q_pos.cuda())
    ok = (idx >= 0) & (idx <= q_pos.view(-1, 1))
    rows = a.float().clone()
    rows[..., :512] += b.float()
    ref = torch.zeros(N, 576).index_add_(0, idx[ok].long(), rows[ok])
    assert torch.allclose(d_lat.cpu(), ref, rtol=1e-5, atol=1e-4)
    K.scatter_add_latent_rows(d_lat, a.cuda(), None, idx.cuda(), q_pos.cuda())          # without the value part
    ref2 = ref + torch.zeros(N, 576).index_add_(0, idx[ok].long(), a.float()[ok])
    assert torch.allclose(d_lat.cpu(), ref2, rtol=1e-5, atol=1e-4)
    assert _lib.read_status(torch.device("cuda")) == 0
    # an index past the destination is skipped and reported
    small = torch.zeros(20, 576, device="cuda")
    K.scatter_add_latent_rows(small, a.cuda(), None, idx.cuda(), torch.full((T,), N, dtype=torch.int32).cuda())
    assert _lib.read_status(torch.device("cuda")) == 2
    ok2 = (idx >= 0) & (idx < 20)
    assert torch.allclose(small.cpu(), torch.zeros(20, 576).index_add_(0, idx[ok2].long(), a.float()[ok2]), rtol=1e-5, atol=1e-4)
