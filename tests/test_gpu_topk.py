"""Top-k kernel against torch.topk / the oracle.  Bit-exact as sets; with distinct scores
also as ordered lists."""
import pytest
import torch

from oracle import dsa_oracle as O

pytestmark = pytest.mark.gpu


def _ref_sets(scores_cpu, k, lo=None, hi=None):
    """Oracle top-k made tie-deterministic: descending score, equal scores by ascending
    position (a stable sort), -1 where the pick is not finite."""
    n_rows, n_cols = scores_cpu.shape
    lo = torch.zeros(n_rows, dtype=torch.int64) if lo is None else lo.long()
    hi = torch.full((n_rows,), n_cols, dtype=torch.int64) if hi is None else hi.long()
    masked = O.mask_interval(scores_cpu, lo, hi)
    vals, order = torch.sort(masked, dim=1, descending=True, stable=True)
    k_eff = min(k, n_cols)
    out = torch.full((n_rows, k), -1, dtype=torch.int32)
    out[:, :k_eff] = torch.where(torch.isfinite(vals[:, :k_eff]), order[:, :k_eff].to(torch.int32),
                                 torch.full((n_rows, k_eff), -1, dtype=torch.int32))
    # same set as the reference's torch.topk (ties aside)
    assert O.set_recall(out, O.topk_rows(masked, k)) > 0.9999
    return out


@pytest.mark.parametrize("n_rows,n_cols,k", [(7, 100, 16), (5, 4096, 2048), (3, 8192, 2048),
                                            (4, 8193, 2048), (2, 131072, 2048), (3, 40000, 512),
                                            (2, 65536, 8192), (9, 33, 64), (1, 1, 1)])
def test_topk_matches_torch(n_rows, n_cols, k):
    from transarch_b200 import kernels as K
    g = torch.Generator().manual_seed(n_cols + k)
    s = torch.randn(n_rows, n_cols, generator=g)
    ref = _ref_sets(s, k)
    idx, val = K.topk_select(s.cuda(), k, return_values=True)
    idx = idx.cpu(); val = val.cpu()
    assert torch.equal(idx, ref)         # randn fp32: distinct values -> same order too
    k_eff = min(k, n_cols)
    assert torch.equal(val[:, :k_eff], torch.gather(s, 1, ref[:, :k_eff].long()))
    assert (idx[:, k_eff:] == -1).all()


def test_topk_ranges_ragged_and_empty():
    from transarch_b200 import kernels as K
    g = torch.Generator().manual_seed(3)
    n_rows, n_cols, k = 12, 20000, 2048
    s = torch.randn(n_rows, n_cols, generator=g)
    lo = torch.randint(0, 5000, (n_rows,), generator=g, dtype=torch.int32)
    hi = torch.randint(5000, n_cols + 1, (n_rows,), generator=g, dtype=torch.int32)
    hi[0] = lo[0]                      # empty row
    hi[1] = lo[1] + 5                  # fewer than k
    hi[2] = lo[2] + 2048               # exactly k
    ref = _ref_sets(s, k, lo, hi)
    idx = K.topk_select(s.cuda(), k, col_begin=lo.cuda(), col_end=hi.cuda()).cpu()
    assert torch.equal(idx, ref)
    assert (idx[0] == -1).all() and (idx[1, 5:] == -1).all() and (idx[2] >= 0).all()


def test_topk_masked_entries_and_inf():
    from transarch_b200 import kernels as K
    g = torch.Generator().manual_seed(4)
    s = torch.randn(6, 8192, generator=g)
    s[:, ::3] = float("-inf")
    s[0, 5] = float("nan")
    s[1, 7] = float("inf")
    idx = K.topk_select(s.cuda(), 4096).cpu()
    for r in range(6):
        row = s[r].clone()
        row[torch.isnan(row) | torch.isinf(row)] = float("-inf")
        n_valid = int(torch.isfinite(row).sum())
        exp = torch.sort(row, descending=True, stable=True).indices[:min(4096, n_valid)]
        assert torch.equal(idx[r, :exp.numel()].long(), exp)
        assert (idx[r, exp.numel():] == -1).all()
    # +inf kept on request, and it sorts first
    idx2 = K.topk_select(s.cuda(), 16, keep_pos_inf=True).cpu()
    assert idx2[1, 0] == 7


def test_topk_massive_ties_take_lowest_positions():
    from transarch_b200 import kernels as K
    # all equal: must select positions 0..k-1 (fallback radix over position bits)
    s = torch.zeros(2, 50000)
    idx = K.topk_select(s.cuda(), 2048).cpu()
    assert torch.equal(idx[0], torch.arange(2048, dtype=torch.int32))
    # two-valued: all the 1.0s (sparse) then the lowest-position 0.0s
    s = torch.zeros(1, 30000)
    ones = torch.arange(0, 30000, 37)
    s[0, ones] = 1.0
    idx = K.topk_select(s.cuda(), 2048).cpu()[0]
    n1 = ones.numel()
    assert torch.equal(idx[:n1].long(), ones)
    rest = [i for i in range(3000) if i % 37 != 0][: 2048 - n1]
    assert idx[n1:].tolist() == rest


def test_topk_position_maps():
    from transarch_b200 import kernels as K
    g = torch.Generator().manual_seed(5)
    n_rows, nblk, P, k = 5, 6, 128, 200
    s = torch.randn(n_rows, nblk * P, generator=g)
    table = torch.stack([torch.randperm(40, generator=g)[:nblk] for _ in range(n_rows)]).to(torch.int32)
    off = torch.tensor([0, -3, 10, 0, 7], dtype=torch.int32)
    idx = K.topk_select(s.cuda(), k, page_table=table.cuda(), page_size=P, row_pos_offset=off.cuda()).cpu()
    cols = torch.topk(s, k, dim=1).indices
    exp = torch.gather(table.long(), 1, cols // P) * P + cols % P + off.view(-1, 1)
    assert torch.equal(idx.long(), exp)
    pm = torch.randint(0, 1 << 20, s.shape, generator=g, dtype=torch.int32)
    idx = K.topk_select(s.cuda(), k, pos_map=pm.cuda()).cpu()
    assert torch.equal(idx, torch.gather(pm, 1, cols))


def test_topk_deterministic_twice():
    from transarch_b200 import kernels as K
    g = torch.Generator().manual_seed(6)
    s = (torch.randn(8, 100000, generator=g) * 4).round() / 4     # many ties
    a = K.topk_select(s.cuda(), 2048)
    b = K.topk_select(s.cuda(), 2048)
    assert torch.equal(a, b)
    # set check against a stable CPU sort: descending value, ascending position
    for r in range(8):
        order = sorted(range(100000), key=lambda i: (-float(s[r, i]), i))[:2048]
        assert a[r].cpu().tolist() == order


@pytest.mark.parametrize("n_cols,k", [(131072, 2048), (5000, 2048), (70000, 8192)])
def test_topk_unsorted_same_set(n_cols, k):
    from transarch_b200 import kernels as K
    g = torch.Generator().manual_seed(n_cols)
    s = torch.randn(3, n_cols, generator=g)
    ref = _ref_sets(s, k)
    idx = K.topk_select(s.cuda(), k, sorted=False).cpu()
    assert torch.equal(torch.sort(idx, dim=1).values, torch.sort(ref, dim=1).values)


@pytest.mark.parametrize("n_rows,n_cols,k,splits", [(5, 131072, 2048, 4), (3, 40000, 512, 3), (64, 32768, 2048, 0),
                                                    (2, 100003, 2048, 7)])
def test_topk_split_equals_single(n_rows, n_cols, k, splits):
    from transarch_b200 import kernels as K
    g = torch.Generator().manual_seed(n_cols * 3 + k)
    s = torch.randn(n_rows, n_cols, generator=g).cuda()
    hi = torch.randint(n_cols // 2, n_cols + 1, (n_rows,), generator=g, dtype=torch.int32)
    hi[0] = 100                                   # a short row: the second kernel selects on its own
    if n_rows > 2:
        hi[2] = 0                                 # an empty row
    off = torch.arange(n_rows, dtype=torch.int32) * 1000
    scratch = K.topk_scratch(n_rows, s.device)
    ref, ref_v = K.topk_select(s, k, col_end=hi.cuda(), row_pos_offset=off.cuda(), return_values=True)
    for _ in range(2):                            # twice: the scratch counters must be re-armed
        out, val = K.topk_select_split(s, k, scratch, col_end=hi.cuda(), row_pos_offset=off.cuda(), splits=splits,
                                       out_values=torch.empty(n_rows, k, device="cuda"))
        assert torch.equal(out, ref) and torch.equal(val, ref_v)
        assert (scratch[1][:n_rows] == 0).all()
    uns = K.topk_select_split(s, k, scratch, col_end=hi.cuda(), row_pos_offset=off.cuda(), sorted=False)
    assert torch.equal(torch.sort(uns, 1).values, torch.sort(ref, 1).values)


def test_topk_split_ties_fall_back():
    from transarch_b200 import kernels as K
    s = torch.zeros(3, 60000, device="cuda")
    s[1] = (torch.arange(60000, device="cuda") % 7).float()
    scratch = K.topk_scratch(3, s.device)
    out = K.topk_select_split(s, 2048, scratch, splits=4)
    assert torch.equal(out, K.topk_select(s, 2048))
    assert torch.equal(out[0].cpu(), torch.arange(2048, dtype=torch.int32))


def test_segments_in_separate_buffers():
    """seg_offsets: the segments of a row live in unrelated allocations (as the candidate buffers of
    peer GPUs do); the result equals the top-k of the concatenated rows."""
    from transarch_b200 import kernels as K
    g = torch.Generator().manual_seed(5)
    rows, k, n_seg = 6, 256, 3
    bufs = []
    for r in range(n_seg):
        pos = torch.stack([torch.randperm(10000, generator=g)[:k] + 10000 * r for _ in range(rows)]).to(torch.int32)
        sc = torch.randn(rows, k, generator=g)
        sc[0, :5] = float("-inf")
        bufs.append(torch.cat([pos, sc.view(torch.int32)], dim=1).cuda().contiguous())   # [rows, 2k]: pos | score bits
    base = bufs[0].data_ptr()
    offs = [(b.data_ptr() - base) // 4 for b in bufs]
    flat = bufs[0].view(-1)
    out = torch.empty(rows, k, dtype=torch.int32, device="cuda")
    K.topk_select(flat[k:].view(torch.float32).view(1, -1), k, sorted=True, pos_map=flat.view(1, -1), out=out,
                  n_cols=n_seg * k, row_stride=2 * k, seg_cols=k, seg_offsets=offs, n_rows=rows, pos_map_stride=2 * k)
    all_pos = torch.cat([b[:, :k] for b in bufs], dim=1).cpu()
    all_sc = torch.cat([b[:, k:].view(torch.float32) for b in bufs], dim=1).cpu()
    for r in range(rows):
        order = sorted(range(n_seg * k), key=lambda c: (-float(all_sc[r, c]), int(all_pos[r, c])))[:k]
        assert out[r].cpu().tolist() == [int(all_pos[r, c]) for c in order]


def test_topk_split_private_list_overflow_falls_back():
    """One collecting thread meets far more candidates than its private list holds (the winners are
    bunched in the columns a single thread of a single slice streams): the row's list is marked
    unusable and the last kernel selects from the row itself.  The result is still exact."""
    from transarch_b200 import kernels as K
    g = torch.Generator().manual_seed(77)
    n_rows, n_cols, k, splits = 4, 131072, 2048, 4
    s = torch.randn(n_rows, n_cols, generator=g)
    # a collecting thread reads 4 consecutive columns out of every 2048 (512 threads x 16-byte loads):
    # 16 such groups inside the first slice of 32768 columns -> 64 winners for that one thread
    cols = (torch.arange(16).view(-1, 1) * 2048 + torch.arange(4).view(1, -1)).reshape(-1)
    s[1, cols] = 10.0 + torch.rand(64, generator=g)
    s[3, cols + 32768 + 4 * 137] = 12.0 + torch.rand(64, generator=g)      # another slice, another thread
    s = s.cuda()
    scratch = K.topk_scratch(n_rows, s.device)
    ref = K.topk_select(s, k)
    for _ in range(3):
        out = K.topk_select_split(s, k, scratch, splits=splits)
        assert torch.equal(out, ref)
        assert (scratch[1][:n_rows] == 0).all()
    assert set(cols.tolist()) <= set(out[1].cpu().tolist())


@pytest.mark.parametrize("n_cols", [700, 3000, 8192, 12000, 16384])
def test_topk_short_rows_ties_and_specials(n_cols):
    """Rows of at most sixteen columns per thread are selected from registers (score keys relative to the
    smallest, then the bit-inverted positions of tied keys): all-equal rows, two-valued rows, coarse values with
    long runs of ties, NaN / -inf / +inf entries, fewer valid scores than k, positions that do not grow with
    the column."""
    from transarch_b200 import kernels as K
    g = torch.Generator().manual_seed(n_cols)
    k = min(2048, n_cols // 2)
    s = torch.zeros(6, n_cols)
    s[1, torch.arange(0, n_cols, 11)] = 1.0                              # two-valued
    s[2] = (torch.randn(n_cols, generator=g) * 3).round() / 2 + 0.0      # coarse: long runs of ties (+ 0.0 turns
                                                                          # -0.0 into +0.0: the keys order the two)
    s[3] = torch.randn(n_cols, generator=g)
    s[3, ::5] = float("nan"); s[3, 1::5] = float("-inf"); s[3, 7] = float("inf")
    s[4] = float("-inf"); s[4, 5:5 + k // 3] = torch.randn(k // 3, generator=g)   # fewer valid scores than k
    s[5] = -torch.arange(n_cols).float()                                  # strictly decreasing
    idx = K.topk_select(s.cuda(), k, sorted=True).cpu()
    un = K.topk_select(s.cuda(), k, sorted=False).cpu()
    for r in range(6):
        row = s[r].clone()
        row[torch.isnan(row) | (row == float("inf"))] = float("-inf")
        n_valid = int(torch.isfinite(row).sum())
        exp = torch.sort(row, descending=True, stable=True).indices[:min(k, n_valid)]
        assert torch.equal(idx[r, :exp.numel()].long(), exp), r
        assert (idx[r, exp.numel():] == -1).all()
        assert torch.equal(torch.sort(un[r]).values, torch.sort(idx[r]).values)
    with_inf = K.topk_select(s.cuda(), 8, keep_pos_inf=True).cpu()
    assert with_inf[3, 0] == 7
    # ties broken by POSITION when positions come from a page table in which they do not grow with the column
    if n_cols % 128 == 0:
        pages = torch.stack([torch.randperm(4 * n_cols // 128, generator=g)[: n_cols // 128] for _ in range(6)]).int()
        got = K.topk_select(s.cuda(), k, page_table=pages.cuda(), page_size=128, sorted=True).cpu()
        col = torch.arange(n_cols)
        pos = pages.long()[:, col // 128] * 128 + (col % 128)
        for r in (0, 1, 2):
            order = sorted(range(n_cols), key=lambda c: (-float(s[r, c]), int(pos[r, c])))[:k]
            assert got[r].tolist() == [int(pos[r, c]) for c in order]
