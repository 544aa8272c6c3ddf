"""The one-kernel peer-memory merge of attention partials.

On one GPU the ranks are emulated one after another without the flag exchange (kernels that wait
for each other must not share a GPU); with two or more GPUs the real exchange runs as one process
per GPU."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _partials(world, n_rows, seed):
    g = torch.Generator().manual_seed(seed)
    ctx = torch.randn(world, n_rows, 512, generator=g).bfloat16()
    lse = 3.0 * torch.randn(world, n_rows, generator=g)
    lse[0, 1] = float("-inf")                      # one empty partial
    lse[:, 2] = float("-inf")                      # a row that is empty on every rank
    if world > 1:
        lse[1, 3] = 40.0                           # one rank dominates
    return ctx, lse


def _expected(ctx, lse):
    m = lse.max(dim=0).values
    w = torch.where(torch.isinf(lse), torch.zeros_like(lse), torch.exp(lse - torch.where(torch.isinf(m), torch.zeros_like(m), m)))
    den = w.sum(0)
    out = (w.unsqueeze(-1) * ctx.float()).sum(0) / den.clamp_min(1e-38).unsqueeze(-1)
    out = torch.where(den.unsqueeze(-1) > 0, out, torch.zeros_like(out))
    lse_out = torch.where(den > 0, m + torch.log(den.clamp_min(1e-38)), torch.full_like(m, float("-inf")))
    return out, lse_out


@pytest.mark.parametrize("world,n_rows", [(4, 1000), (2, 8192), (8, 37), (1, 64)])
def test_emulated_ranks_one_after_another(world, n_rows):
    from transarch_b200 import _lib
    from transarch_b200.peer import PeerLseCombine
    dev = torch.device("cuda")
    pc = PeerLseCombine(n_rows, dev, emulate_world=world)
    try:
        for step in range(2):                                   # the step counter advances by itself
            ctx, lse = _partials(world, n_rows, 7 + step)
            for r in range(world):
                c, l, o, lo = pc.views_of(r)
                c.copy_(ctx[r]); l.copy_(lse[r]); o.fill_(7.0); lo.fill_(7.0)
            for r in range(world):
                pc.run(rank=r, no_sync=True)
            torch.cuda.synchronize()
            want, want_lse = _expected(ctx, lse)
            for r in range(world):
                _, _, o, lo = pc.views_of(r)
                assert torch.allclose(o.float().cpu(), want, rtol=1e-2, atol=1e-2)
                assert torch.allclose(lo.cpu(), want_lse, rtol=1e-5, atol=1e-5)
                assert (o[2] == 0).all()
            assert [int(s[0]) for s in pc.state] == [step + 1] * world
        # reduce-scatter form: each rank keeps only its own slice of the rows, in its own buffer
        for r in range(world):
            _, _, o, lo = pc.views_of(r)
            o.fill_(7.0); lo.fill_(7.0)
        for r in range(world):
            pc.run(rank=r, no_sync=True, local_only=True)
        torch.cuda.synchronize()
        for r in range(world):
            a, b = pc.row_slice(r)
            _, _, o, lo = pc.views_of(r)
            assert torch.allclose(o[a:b].float().cpu(), want[a:b], rtol=1e-2, atol=1e-2)
            assert torch.allclose(lo[a:b].cpu(), want_lse[a:b], rtol=1e-5, atol=1e-5)
            assert (o[:a] == 7).all() and (o[b:] == 7).all()
        assert _lib.read_status(dev) == 0
    finally:
        pc.close()


def test_wait_for_absent_peer_runs_out_and_is_reported():
    """A bounded device wait that really runs out, on one GPU and without any fault: a barrier for a
    world of two over two local buffers where nobody ever plays rank 1.  With the limit lowered to
    about a millisecond the kernel must come back, raise the status word to 1 and advance its step
    counter; the stream stays usable and a following ordinary call gives correct results."""
    import time
    from transarch_b200 import _lib
    from transarch_b200.peer import PeerLseCombine
    lib = _lib.load()
    dev = torch.device("cuda")
    n_rows = 64
    pc = PeerLseCombine(n_rows, dev, emulate_world=2, extra_bytes=3 * 1024)
    assert _lib.read_status(dev) == 0
    assert lib.b200dsa_peer_set_wait_limit(1 << 21) == 0          # ~1 ms at 2 GHz
    try:
        t0 = time.perf_counter()
        pc.barrier(slot=1)                                        # rank 0 of 2; rank 1's flag never arrives
        torch.cuda.synchronize()
        assert time.perf_counter() - t0 < 5.0
        assert _lib.read_status(dev) == 1                         # reported (and cleared by the read)
        assert int(pc.barrier_state[0]) == 1                      # the step counter still advanced
        pc.push_extra(1024, slot=3)                               # the all-gather kernel gives up the same way
        torch.cuda.synchronize()
        assert _lib.read_status(dev) == 1
    finally:
        assert lib.b200dsa_peer_set_wait_limit(0) == 0            # back to the default
    # the context is intact: an ordinary (emulated, no waiting) merge on the same buffers is correct
    ctx, lse = _partials(2, n_rows, 3)
    for r in range(2):
        c, l, o, lo = pc.views_of(r)
        c.copy_(ctx[r]); l.copy_(lse[r])
    for r in range(2):
        pc.run(rank=r, no_sync=True)
    torch.cuda.synchronize()
    want, want_lse = _expected(ctx, lse)
    assert torch.allclose(pc.views_of(0)[2].float().cpu(), want, rtol=1e-2, atol=1e-2)
    assert torch.allclose(pc.views_of(1)[3].cpu(), want_lse, rtol=1e-5, atol=1e-5)
    assert _lib.read_status(dev) == 0
    assert lib.b200dsa_peer_set_wait_limit(-1) == -1              # rejected
    pc.close()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _sharded_step_agrees(rank, world, dev):
    """The whole key-sharded step with the exchanges in peer memory against the same step through
    NCCL: identical selection, same context up to bf16 rounding."""
    from transarch_b200 import _lib
    from transarch_b200.decode import ShardInfo, SparseDecodeStep
    from transarch_b200.workloads import make_decode_queries, make_decode_state
    B, ctx_len, topk = 8, 16384, 2048
    shard_len = ctx_len // world
    shard = ShardInfo(rank=rank, world_size=world, shard_len=shard_len)
    st = make_decode_state(B, ctx_len, page_size=64, seed=5, rank=rank, world_size=world, shard_len=shard_len,
                           device=dev)
    res = {}
    for mode in ("peer", "nccl"):
        step = SparseDecodeStep(B, shard_len, topk=topk, device=dev, shard=shard, sorted_topk=True, combine=mode)
        assert (step.peer is not None) == (mode == "peer")
        for i in range(2):                                        # twice: flags and step counters advance
            q_idx, w, q_lat = make_decode_queries(B, 128, seed=40 + i, device=dev)
            idx, c, lse = step.run(q_idx, w, q_lat, st.k_cache, st.context_lens, st.block_table, st.kv,
                                   st.kv_row_base, st.context_lens_local)
            torch.cuda.synchronize()
            res[mode, i] = (idx.clone(), c.float().clone(), lse.clone())
        if step.peer is not None:
            import torch.distributed as dist
            dist.barrier()
            step.peer.close()
    ok = _lib.read_status(dev) == 0
    for i in range(2):
        a, b = res["peer", i], res["nccl", i]
        ok = ok and torch.equal(a[0], b[0]) and torch.allclose(a[1], b[1], rtol=2e-2, atol=2e-2) and \
            torch.allclose(a[2], b[2], rtol=1e-4, atol=1e-4)
    return ok


def _rank_main(rank, world, port, ret):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from transarch_b200 import _lib
        from transarch_b200.peer import PeerLseCombine
        n_rows = 8192
        pc = PeerLseCombine(n_rows, dev)
        ok = True
        for step in range(3):
            ctx, lse = _partials(world, n_rows, 21 + step)
            pc.ctx.copy_(ctx[rank]); pc.lse.copy_(lse[rank])
            out, lse_out = pc.run()
            torch.cuda.synchronize()
            want, want_lse = _expected(ctx, lse)
            ok = ok and torch.allclose(out.float().cpu(), want, rtol=1e-2, atol=1e-2) and \
                torch.allclose(lse_out.cpu(), want_lse, rtol=1e-5, atol=1e-5)
        ok = ok and _lib.read_status(dev) == 0
        dist.barrier()
        pc.close()
        ok = ok and _sharded_step_agrees(rank, world, dev)
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpus_exchange_over_peer_memory():
    import torch.multiprocessing as mp
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    ctx = mp.get_context("spawn")
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=180)
    stuck = [p for p in procs if p.is_alive()]
    for p in stuck:
        p.kill()
    assert not stuck, "a rank did not finish"
    assert ret.get(0) is True and ret.get(1) is True


def test_folded_exchanges_on_one_gpu():
    """The three kernels that carry the exchanges of the key-sharded step, checked on one GPU with the
    two ranks' buffers as two local allocations (nothing waits): the selection's push lands in every
    buffer's receive slot and raises the flag; the merge of pushed lists equals top-k + compaction; the
    attention kernel raises the merge kernel's "ready" flag without changing its results."""
    from transarch_b200 import _lib, kernels as K
    from transarch_b200.peer import PeerLseCombine
    from transarch_b200.workloads import make_decode_state
    dev = torch.device("cuda")
    B, k, H, world = 5, 256, 128, 2
    ctxs = [3000, 9000, 700, 100, 0]
    st = make_decode_state(B, ctxs, page_size=64, seed=11)
    g = torch.Generator().manual_seed(11)
    q = torch.randn(B, 64, 128, generator=g).bfloat16().cuda()
    w = (torch.randn(B, 64, generator=g) / 8).cuda()
    q_fp8, wf = K.quant_q_fold_weights(q, w, 128 ** -0.5)
    cand_bytes = B * 2 * k * 4
    pc = PeerLseCombine(B * H, dev, emulate_world=world, extra_bytes=cand_bytes * (1 + world))
    try:
        scratch = K.fused_scratch(B, dev)
        off = torch.full((B,), 1000, dtype=torch.int32, device=dev)
        ref_idx, ref_val = K.indexer_paged_fp8_topk(q_fp8, wf, st.k_cache, 64, st.context_lens, st.block_table, k,
                                                    scratch, max_cols=st.local_len, row_pos_offset=off, sorted=True,
                                                    out_values=torch.empty(B, k, device=dev))
        link = pc.link(1)                                               # rank 0 of 2
        for rep in range(2):
            idx, val = K.indexer_paged_fp8_topk(q_fp8, wf, st.k_cache, 64, st.context_lens, st.block_table, k, scratch,
                                                max_cols=st.local_len, row_pos_offset=off, sorted=True,
                                                out_values=torch.empty(B, k, device=dev),
                                                push=(link, pc.off_extra + cand_bytes))
            torch.cuda.synchronize()
            assert torch.equal(idx, ref_idx) and torch.equal(val, ref_val)
            for r in range(world):                                      # slot 0 (this rank) of both receive areas
                recv = pc.extra_of(r)[cand_bytes:].view(torch.int32).view(world, B, 2 * k)
                assert torch.equal(recv[0, :, :k], ref_idx)
                assert torch.equal(recv[0, :, k:].view(torch.float32), ref_val)
                flags = pc.buffers.views[r][pc.off_flags:pc.off_flags + 256].view(torch.int32)
                assert int(flags[1 * 8 + 0]) == rep + 1                 # flag word slot 1, written by rank 0
            assert int(pc.barrier_state[0]) == rep + 1 and int(pc.barrier_state[1]) == 0
        # ---- merge of pushed lists (no link: nothing to wait for) against select + compaction
        recv = torch.empty(world, B, 2 * k, dtype=torch.int32, device=dev)
        for r in range(world):
            pos = torch.stack([torch.randperm(5000, generator=g)[:k] + 5000 * r for _ in range(B)]).to(torch.int32)
            sc = torch.randn(B, k, generator=g)
            sc[0, :7] = float("-inf"); pos[0, :7] = -1
            recv[r, :, :k] = pos.cuda(); recv[r, :, k:] = sc.view(torch.int32).cuda()
        merged = torch.empty(B, k, dtype=torch.int32, device=dev)
        owned = torch.empty(B, k, dtype=torch.int32, device=dev)
        cnt = torch.empty(B, dtype=torch.int32, device=dev)
        K.topk_merge_owned(recv, k, 5000, 10000, out=merged, owned=owned, owned_count=cnt, sorted=True)
        flat = recv.view(-1)
        want = K.topk_select(flat[k:].view(torch.float32).view(1, -1), k, sorted=True, pos_map=flat.view(1, -1),
                             n_cols=world * k, row_stride=2 * k, seg_cols=k, seg_stride=B * 2 * k, n_rows=B,
                             pos_map_stride=2 * k)
        assert torch.equal(merged, want)
        for b in range(B):
            own = want[b][(want[b] >= 5000) & (want[b] < 10000)]
            assert int(cnt[b]) == own.numel()
            assert torch.equal(torch.sort(owned[b, :own.numel()]).values, torch.sort(own).values)
            assert (owned[b, own.numel():] == -1).all()
        # ---- attention raising the merge kernel's "ready" flag
        kv = (0.5 * torch.randn(2000, 576, generator=g)).bfloat16().cuda()
        q_lat = torch.randn(B, H, 576, generator=g).bfloat16().cuda()
        sel = torch.stack([torch.randperm(2000, generator=g)[:k] for _ in range(B)]).to(torch.int32).cuda()
        c0, l0 = K.sparse_mla_decode(q_lat, kv, sel, 192 ** -0.5)
        c0, l0 = c0.clone(), l0.clone()
        c1, l1 = K.sparse_mla_decode(q_lat, kv, sel, 192 ** -0.5, signal=(pc.link(0), pc.ticket))
        torch.cuda.synchronize()
        assert torch.equal(c0, c1) and torch.equal(l0, l1)
        for r in range(world):
            flags = pc.buffers.views[r][pc.off_flags:pc.off_flags + 256].view(torch.int32)
            assert int(flags[0]) == int(pc.state[0][0]) + 1             # "ready" word of rank 0, next step
        assert int(pc.ticket) == 0
        assert _lib.read_status(dev) == 0
    finally:
        pc.close()
