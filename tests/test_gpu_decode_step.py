"""Whole decode step (quantise q -> indexer -> top-k -> sparse MLA) against the oracle, and
the key-sharded flow emulated on one GPU (two shards run one after the other, the all-gather
replaced by a copy) against the unsharded result."""
import pytest
import torch

from oracle import dsa_oracle as O
from tests.decode_cases import make_global_problem, oracle_decode, shard_state

pytestmark = pytest.mark.gpu
IDX_SCALE, ATT_SCALE = 128 ** -0.5, 192 ** -0.5


def _cuda(prob):
    return prob["q_idx"].cuda(), prob["w"].cuda(), prob["q_lat"].cuda()


@pytest.mark.parametrize("ctxs,topk", [([3000, 8192, 700, 5555], 512), ([20000, 9000], 2048)])
def test_single_gpu_step_matches_oracle(ctxs, topk):
    from transarch_b200 import _lib
    from transarch_b200.decode import SparseDecodeStep
    prob = make_global_problem(41, ctxs)
    st = shard_state(prob, 0, 1, max(ctxs), "cuda")
    step = SparseDecodeStep(len(ctxs), st["table"].shape[1] * 64, topk=topk, sorted_topk=True)
    q_idx, w, q_lat = _cuda(prob)
    idx, ctx, lse = step.run(q_idx, w, q_lat, st["cache"], st["lens"], st["table"], st["kv"], st["base"])
    assert _lib.read_status(ctx.device) == 0
    ref_idx, scores, ref_ctx, ref_lse = oracle_decode(prob, topk, IDX_SCALE, ATT_SCALE)
    idx = idx.cpu()
    assert O.set_recall(idx, ref_idx) >= 0.999
    total, bad = O.near_tie_audit(idx, ref_idx, torch.cat([torch.nn.functional.pad(s, (0, max(ctxs) - s.shape[1]),
                                  value=float("-inf")) for s in scores]), rtol=1e-3)
    assert bad == 0, f"{bad} of {total} disagreements are not near-ties"
    # attention compared on the kernel's own selection (removes tie effects)
    for b in range(len(ctxs)):
        c, l = O.sparse_attend_latent(prob["q_lat"][b:b + 1], prob["kv"][b], idx[b:b + 1], d_c=512,
                                      sm_scale=ATT_SCALE, q_pos=torch.tensor([ctxs[b] - 1]))
        err = (ctx[b].cpu() - c[0]).abs().max() / c.abs().max()
        assert err < 2e-2
        assert (lse[b].cpu() - l[0]).abs().max() < 2e-2
    err = (ctx.cpu() - ref_ctx).abs().max() / ref_ctx.abs().max()
    assert err < 2e-2


def test_two_shards_equal_unsharded():
    from transarch_b200 import kernels as K
    from transarch_b200.decode import ShardInfo, SparseDecodeStep
    ctxs, topk, shard_len = [6000, 8192, 2500], 1024, 4096
    prob = make_global_problem(42, ctxs)
    q_idx, w, q_lat = _cuda(prob)
    full = shard_state(prob, 0, 1, max(ctxs), "cuda")
    one = SparseDecodeStep(3, full["table"].shape[1] * 64, topk=topk, sorted_topk=True)
    idx1, ctx1, lse1 = one.run(q_idx, w, q_lat, full["cache"], full["lens"], full["table"], full["kv"], full["base"])
    idx1, ctx1, lse1 = idx1.clone(), ctx1.clone(), lse1.clone()

    steps, states = [], []
    for r in range(2):
        st = shard_state(prob, r, 2, shard_len, "cuda")
        sp = SparseDecodeStep(3, shard_len, topk=topk, sorted_topk=True,
                              shard=ShardInfo(rank=r, world_size=2, shard_len=shard_len))
        sp.select(q_idx, w, st["cache"], st["local"], st["table"])
        steps.append(sp); states.append(st)
    gathered = torch.stack([s.cand for s in steps])            # what the all-gather delivers
    parts, lses = [], []
    for r, sp in enumerate(steps):
        sp.cand_all.copy_(gathered)
        flat = sp.cand_all.view(-1)
        K.topk_select(flat[topk:].view(torch.float32).view(1, -1), topk, sorted=True, pos_map=flat.view(1, -1),
                      out=sp.merged, n_cols=2 * topk, row_stride=2 * topk, seg_cols=topk,
                      seg_stride=3 * 2 * topk, n_rows=3, pos_map_stride=2 * topk)
        assert torch.equal(sp.merged, idx1), "merged shard candidates differ from the unsharded top-k"
        torch.sub(states[r]["lens"], 1, out=sp.q_pos)
        c, l = sp.attend(q_lat, states[r]["kv"], states[r]["base"], sp.merged, sp.q_pos)
        parts.append(c.clone()); lses.append(l.clone())
    ctx2, lse2 = K.lse_combine(torch.stack(parts), torch.stack(lses))
    assert (ctx2 - ctx1).abs().max() / ctx1.abs().max() < 2e-3
    assert (lse2 - lse1).abs().max() < 2e-3
    # all-reduce form: prescale with the max, sum, finalize
    m = torch.maximum(lses[0], lses[1])
    wire = sum(K.lse_prescale(parts[r], lses[r], m, torch.empty(3 * 128, K.WIRE_ROW, device="cuda")) for r in range(2))
    ctx3, lse3 = K.lse_finalize(wire.contiguous(), m, torch.empty_like(ctx1), torch.empty_like(lse1))
    assert (ctx3 - ctx2).abs().max() < 1e-5 and (lse3 - lse2).abs().max() < 1e-5


def test_quant_fold_matches_oracle_bitwise():
    from transarch_b200 import kernels as K
    g = torch.Generator().manual_seed(9)
    q = torch.randn(37, 64, 128, generator=g).bfloat16()
    q[3, 5] = 0                                                  # all-zero head: scale floor
    w = torch.randn(37, 64, generator=g) / 8
    q_fp8, wf = K.quant_q_fold_weights(q.cuda(), w.cuda(), IDX_SCALE)
    rq, rw = O.quant_q_fold_weights(q.float(), w, IDX_SCALE)
    assert torch.equal(q_fp8.cpu().view(torch.uint8), rq.view(torch.uint8))
    assert torch.allclose(wf.cpu(), rw, rtol=1e-6, atol=0)


def test_compact_owned():
    from transarch_b200 import kernels as K
    g = torch.Generator().manual_seed(12)
    idx = torch.randint(-1, 5000, (7, 2048), generator=g, dtype=torch.int32)
    out = torch.empty_like(idx).cuda(); cnt = torch.empty(7, dtype=torch.int32, device="cuda")
    K.compact_owned(idx.cuda(), 1000, 2500, out, cnt)
    for r in range(7):
        own = idx[r][(idx[r] >= 1000) & (idx[r] < 2500)]
        assert int(cnt[r]) == own.numel()
        assert torch.equal(out[r, :own.numel()].cpu(), own) and (out[r, own.numel():] == -1).all()


def test_prescale_norm_equals_combine():
    from transarch_b200 import kernels as K
    g = torch.Generator().manual_seed(13)
    R, n, H = 4, 3, 16
    parts = torch.randn(R, n, H, 512, generator=g).cuda()
    lses = torch.randn(R, n, H, generator=g).cuda() * 3
    lses[2, 1] = float("-inf")                       # an empty partial
    lses[:, 2, 5] = float("-inf")                    # a row empty on every rank
    ref_ctx, ref_lse = K.lse_combine(parts, lses)
    acc = torch.zeros(n, H, 512, device="cuda")
    for r in range(R):
        out = torch.empty(n, H, 512, dtype=torch.bfloat16, device="cuda")
        lse_out = torch.empty(n, H, device="cuda")
        K.lse_prescale_norm(parts[r].contiguous(), lses, r, out, lse_out)
        acc += out.float()
        assert torch.equal(torch.isfinite(lse_out), torch.isfinite(ref_lse))
        fin = torch.isfinite(ref_lse)
        assert (lse_out[fin] - ref_lse[fin]).abs().max() < 1e-5
    assert (acc - ref_ctx).abs().max() < 2e-2 * ref_ctx.abs().max()
    assert (acc[2, 5] == 0).all()


@pytest.mark.parametrize("world", [4, 8])
def test_many_shards_through_peer_buffers_emulated(world):
    """The peer-memory data path with 4 and 8 shards on one GPU: every shard's candidates and
    partials live in their own exchange buffer, the merge reads them through per-segment offsets and
    the one-kernel combine runs rank after rank without the flag exchange.  Result: the unsharded one."""
    from transarch_b200 import _lib
    from transarch_b200.decode import ShardInfo, SparseDecodeStep
    from transarch_b200.peer import PeerLseCombine
    shard_len, topk, H = 1024, 512, 128
    ctxs = [world * shard_len, world * shard_len - 700, 3 * shard_len + 5]
    B = len(ctxs)
    prob = make_global_problem(43, ctxs)
    q_idx, w, q_lat = _cuda(prob)
    full = shard_state(prob, 0, 1, max(ctxs), "cuda")
    one = SparseDecodeStep(B, full["table"].shape[1] * 64, topk=topk, sorted_topk=True)
    idx1, ctx1, lse1 = [t.clone() for t in one.run(q_idx, w, q_lat, full["cache"], full["lens"], full["table"],
                                                     full["kv"], full["base"])]
    dev = torch.device("cuda")
    pc = PeerLseCombine(B * H, dev, emulate_world=world, extra_bytes=B * 2 * topk * 4)
    try:
        steps, states = [], []
        for r in range(world):
            st = shard_state(prob, r, world, shard_len, "cuda")
            sp = SparseDecodeStep(B, shard_len, topk=topk, sorted_topk=True,
                                  shard=ShardInfo(rank=r, world_size=world, shard_len=shard_len))
            c, l, _, _ = pc.views_of(r)                   # what SparseDecodeStep does with a real group
            sp.ctx, sp.lse = c.view(B, H, 512), l.view(B, H)
            sp.cand = pc.extra_of(r).view(torch.int32).view(B, 2 * topk)
            sp.select(q_idx, w, st["cache"], st["local"], st["table"])
            steps.append(sp); states.append(st)
        base = pc.buffers.addresses
        for r, sp in enumerate(steps):
            flat = sp.cand.view(-1)
            sp.K.topk_select(flat[topk:].view(torch.float32).view(1, -1), topk, sorted=True, pos_map=flat.view(1, -1),
                             out=sp.merged, n_cols=world * topk, row_stride=2 * topk, seg_cols=topk,
                             seg_offsets=[(a - base[r]) // 4 for a in base], n_rows=B, pos_map_stride=2 * topk)
            assert torch.equal(sp.merged, idx1), "merged shard candidates differ from the unsharded top-k"
            torch.sub(states[r]["lens"], 1, out=sp.q_pos)
            sp.attend(q_lat, states[r]["kv"], states[r]["base"], sp.merged, sp.q_pos)
        for r in range(world):
            pc.run(rank=r, no_sync=True)
        torch.cuda.synchronize()
        assert _lib.read_status(dev) == 0
        for r in range(world):
            _, _, out, lse_out = pc.views_of(r)
            err = (out.float().view(B, H, 512) - ctx1.float()).abs().max() / ctx1.float().abs().max()
            assert err < 2e-2
            assert (lse_out.view(B, H) - lse1).abs().max() < 1e-3
    finally:
        pc.close()


def test_pipelined_decode_returns_each_steps_own_result():
    """Two captured steps used in turn with host buffers: every submitted input set comes back with the result
    the eager step gives for it (no slot hands out another step's data, inputs are not overwritten early)."""
    from transarch_b200 import _lib
    from transarch_b200.decode import GraphedDecodeStep, PipelinedDecode, SparseDecodeStep, pack_inputs
    ctxs = [6000, 9000, 3000]
    prob = make_global_problem(43, ctxs)
    st = shard_state(prob, 0, 1, max(ctxs), "cuda")
    args = (st["cache"], st["lens"], st["table"], st["kv"], st["base"])
    mk = lambda: SparseDecodeStep(len(ctxs), st["table"].shape[1] * 64, topk=512, sorted_topk=True,
                                  ctx_dtype=torch.bfloat16)
    eager = mk()
    graphs = []
    for _ in range(2):
        stp = mk()
        stp.run(*_cuda(prob), *args)
        torch.cuda.synchronize()
        graphs.append(GraphedDecodeStep(stp, *args).capture())
    pipe = PipelinedDecode(graphs)
    g = torch.Generator().manual_seed(7)
    sets, want = [], []
    for i in range(5):
        q_idx = torch.randn(prob["q_idx"].shape, generator=g).bfloat16()
        w = (torch.randn(prob["w"].shape, generator=g) / 8).float()
        q_lat = torch.randn(prob["q_lat"].shape, generator=g).bfloat16()
        sets.append(pack_inputs(q_idx, w, q_lat).pin_memory())
        idx, ctx, _ = eager.run(q_idx.cuda(), w.cuda(), q_lat.cuda(), *args)
        want.append((idx.cpu().clone(), ctx.cpu().clone()))
    slots = []
    for i in range(5):
        sl = pipe.submit(sets[i])
        slots.append(sl)
        if i >= 1:                                # read step i-1 while step i is in flight
            idx, ctx = pipe.result(slots[i - 1])
            assert torch.equal(idx, want[i - 1][0]) and torch.equal(ctx, want[i - 1][1])
    idx, ctx = pipe.result(slots[4])
    assert torch.equal(idx, want[4][0]) and torch.equal(ctx, want[4][1])
    assert _lib.read_status(torch.device("cuda")) == 0
