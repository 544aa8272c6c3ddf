"""Key-sharded decode step on two CPU ranks (gloo): the host logic of SparseDecodeStep — shard
ranges, candidate wire layout, all-gather + segmented merge, log-sum-exp all-reduce — must give
every rank the unsharded oracle result.  Kernels are replaced by the oracle-backed stand-in."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tests.decode_cases import make_global_problem, oracle_decode, shard_state

CTXS, TOPK, SHARD = [700, 1024, 130], 128, 512


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def _worker(rank, world, port, wire, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from tests import cpu_backend
        from transarch_b200.decode import ShardInfo, SparseDecodeStep, local_context_lens
        torch.set_num_threads(2)
        prob = make_global_problem(51, CTXS, H=8)
        st = shard_state(prob, rank, world, SHARD, "cpu")
        shard = ShardInfo(rank=rank, world_size=world, shard_len=SHARD)
        assert torch.equal(local_context_lens(st["lens"], shard), st["local"])
        step = SparseDecodeStep(len(CTXS), SHARD, topk=TOPK, n_heads=8, device=torch.device("cpu"), shard=shard,
                                backend=cpu_backend, sorted_topk=True, wire=wire)
        idx, ctx, lse = step.run(prob["q_idx"], prob["w"], prob["q_lat"], st["cache"], st["lens"], st["table"],
                                 st["kv"], st["base"])
        ref_idx, _, ref_ctx, ref_lse = oracle_decode(prob, TOPK, 128 ** -0.5, 192 ** -0.5)
        tol = dict(rtol=1e-4, atol=1e-5) if wire == "fp32" else dict(rtol=2e-2, atol=2e-3)   # bf16 wire
        want = torch.bfloat16 if wire == "bf16" else torch.float32       # the wire that was asked for ran
        ok = ctx.dtype == want and torch.equal(idx, ref_idx) and torch.allclose(ctx.float(), ref_ctx, **tol) and \
            torch.allclose(lse, ref_lse, rtol=1e-4, atol=1e-5)
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("wire", ["fp32", "bf16"])
def test_two_rank_sharded_step_matches_unsharded(wire):
    port = _free_port()
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(2, port, wire, ret), nprocs=2, join=True)
    assert ret.get(0) is True and ret.get(1) is True


def _absent_worker(rank, world, port, ret):
    """Both ranks complete one sharded step; then rank 1 leaves between steps with nothing in flight.
    Rank 0's next step must end with an error from its first exchange (short process-group
    timeout) instead of hanging, and must not hand back a result."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import datetime
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    try:
        from tests import cpu_backend
        from transarch_b200.decode import ShardInfo, SparseDecodeStep
        torch.set_num_threads(2)
        prob = make_global_problem(52, CTXS, H=8)
        st = shard_state(prob, rank, world, SHARD, "cpu")
        shard = ShardInfo(rank=rank, world_size=world, shard_len=SHARD)
        step = SparseDecodeStep(len(CTXS), SHARD, topk=TOPK, n_heads=8, device=torch.device("cpu"), shard=shard,
                                backend=cpu_backend, sorted_topk=True, wire="fp32")
        args = (prob["q_idx"], prob["w"], prob["q_lat"], st["cache"], st["lens"], st["table"], st["kv"], st["base"])
        idx, _, _ = step.run(*args)
        ref_idx, _, _, _ = oracle_decode(prob, TOPK, 128 ** -0.5, 192 ** -0.5)
        first_ok = torch.equal(idx, ref_idx)
        if rank == 1:
            ret[1] = "left" if first_ok else "wrong first step"
            return                      # leaves between steps
        try:
            step.run(*args)
            ret[0] = "no error"
        except Exception:               # noqa: BLE001 - the collective's timeout / peer-closed error
            ret[0] = "error" if first_ok else "wrong first step"
    finally:
        try:
            dist.destroy_process_group()
        except Exception:               # noqa: BLE001
            pass


def test_rank_leaving_between_steps_fails_the_next_step_not_hangs():
    port = _free_port()
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_absent_worker, args=(2, port, ret), nprocs=2, join=True)
    assert ret.get(0) == "error" and ret.get(1) == "left"
