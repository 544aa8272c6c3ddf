"""The row-in-shared-memory selection that b200dsa_topk_select uses for many rows (at least 256 rows of at most
8192 columns, k up to 4096), against a stable sort and against the large one-CTA-per-row kernel (reached through
a row count below the switch): same sets, same order."""
import pytest
import torch

from oracle import dsa_oracle as O

pytestmark = pytest.mark.gpu


def _ref_sorted(scores, k, begin=None, end=None, keep_inf=False):
    s = scores.clone()
    n = s.shape[1]
    col = torch.arange(n).view(1, -1)
    if begin is not None:
        s[col < begin.view(-1, 1)] = float("-inf")
    if end is not None:
        s[col >= end.view(-1, 1)] = float("-inf")
    s[torch.isnan(s)] = float("-inf")
    if not keep_inf:
        s[s == float("inf")] = float("-inf")
    # stable descending sort: equal scores keep ascending position, the rule of the kernels (torch.topk, which
    # the reference calls, leaves the order of ties unspecified)
    vals, idx = torch.sort(s, dim=1, descending=True, stable=True)
    kk = min(k, n)
    out = torch.full((s.shape[0], k), -1, dtype=torch.int32)
    out[:, :kk] = torch.where(torch.isfinite(vals[:, :kk]) | (keep_inf & (vals[:, :kk] == float("inf"))),
                              idx[:, :kk].int(), torch.full_like(idx[:, :kk], -1).int())
    return out


@pytest.mark.parametrize("n_rows,n_cols,k", [(4100, 4096, 2048), (1100, 1024, 64), (1030, 700, 1000), (3100, 3000, 256),
                                             (1024, 90, 200), (1500, 1024, 4096), (300, 8192, 2048), (256, 8190, 4096)])
def test_many_rows_match_the_oracle(n_rows, n_cols, k):
    from transarch_b200 import kernels as K
    g = torch.Generator().manual_seed(n_cols + k)
    s = torch.randn(n_rows, n_cols, generator=g)
    s[3, ::7] = float("nan")
    s[4, 5:50] = float("-inf")
    s[5, 10] = float("inf")
    end = torch.randint(1, n_cols + 1, (n_rows,), generator=g, dtype=torch.int32)
    begin = (end.float() * torch.rand(n_rows, generator=g) * 0.3).int()
    end[7] = begin[7]                                   # an empty row
    got = K.topk_select(s.cuda(), k, col_begin=begin.cuda(), col_end=end.cuda(), sorted=True).cpu()
    ref = _ref_sorted(s, k, begin, end)
    assert torch.equal(got, ref)
    un = K.topk_select(s.cuda(), k, col_begin=begin.cuda(), col_end=end.cuda(), sorted=False).cpu()
    assert torch.equal(torch.sort(un, dim=1).values, torch.sort(ref, dim=1).values)
    idx, val = K.topk_select(s.cuda(), k, col_begin=begin.cuda(), col_end=end.cuda(), sorted=True, return_values=True)
    ok = idx.cpu() >= 0
    assert torch.equal(val.cpu()[ok], torch.gather(s, 1, idx.cpu().clamp(min=0).long())[ok])
    assert torch.isinf(val.cpu()[~ok]).all()


@pytest.mark.parametrize("k", [700, 200])
def test_many_rows_massive_ties_and_position_maps(k):
    """Ties are broken towards the lowest POSITION, also when positions come from a page table in which
    they do not grow with the column; thousands of exactly equal scores (zeros) around the threshold."""
    from transarch_b200 import kernels as K
    g = torch.Generator().manual_seed(5)
    n_rows, n_cols = 2100, 2048
    s = torch.zeros(n_rows, n_cols)
    hot = torch.rand(n_rows, n_cols, generator=g) < 0.2
    s[hot] = torch.randn(int(hot.sum()), generator=g).abs()      # about 400 positive scores, the rest exact zeros
    s[:, 100:140] = 0.5                                           # a run of equal positive scores as well
    pages = torch.stack([torch.randperm(64, generator=g)[:16] for _ in range(n_rows)]).int()   # 16 pages of 128
    got = K.topk_select(s.cuda(), k, page_table=pages.cuda(), page_size=128, sorted=True).cpu()
    few = K.topk_select(s[:40].cuda(), k, page_table=pages[:40].cuda(), page_size=128, sorted=True).cpu()  # large CTA per row
    assert torch.equal(got[:40], few)
    col = torch.arange(n_cols)
    pos = pages.long()[:, col // 128] * 128 + (col % 128)
    # reference: sort by (score desc, position asc)
    for r in (0, 17, 2099):
        order = sorted(range(n_cols), key=lambda c: (-float(s[r, c]), int(pos[r, c])))[:k]
        assert got[r].tolist() == [int(pos[r, c]) for c in order]
    un = K.topk_select(s.cuda(), k, page_table=pages.cuda(), page_size=128, sorted=False).cpu()
    assert torch.equal(torch.sort(un, dim=1).values, torch.sort(got, dim=1).values)
    # plain columns
    a = K.topk_select(s.cuda(), k, sorted=True).cpu()
    b = K.topk_select(s[:40].cuda(), k, sorted=True).cpu()
    assert torch.equal(a[:40], b)
    assert torch.equal(a, _ref_sorted(s, k))
