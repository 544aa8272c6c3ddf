"""Sparse decode step: indexer logits -> top-k -> (key-sharded merge) -> sparse MLA attention
-> (log-sum-exp combine).

Single GPU: three launches on pre-allocated buffers, nothing is allocated per step.

Key-sharded over N ranks of one box (keys of every request split into N contiguous position
ranges; rank r owns [r*shard_len, (r+1)*shard_len)): every rank scores and selects inside
its own range, the per-rank candidate lists (global position, score) are all-gathered,
every rank selects the same global top-k from the N*k candidates (the union of the shard
top-k contains the global top-k; ties resolve towards the lowest global position on every
rank alike), attends the selected keys it owns, and the partial (context, lse) pairs are
merged: all-gather of lse (4 B per row), normalised bf16 shares, one SUM all-reduce of the bf16
rows (or, with wire="fp32": MAX all-reduce of lse, pre-scale, SUM all-reduce of 516-wide fp32
rows, divide).
The query-side inputs are replicated.  The reference has no such path; the idea of local
queries against position-indexed keys follows OpenDSA's context-parallel forward
(OpenDSA/opendsa/modeling/dsa_attention.py:620-684).

`backend` is the module providing the kernel wrappers (transarch_b200.kernels by default).
Host-logic tests on CPU ranks pass a stand-in with the same function names.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence, Tuple

import torch
import torch.distributed as dist


@dataclass
class ShardInfo:
    rank: int = 0
    world_size: int = 1
    shard_len: int = 0          # positions per rank (0 = unsharded)
    group: Optional[object] = None

    @property
    def pos_lo(self) -> int:
        return self.rank * self.shard_len if self.world_size > 1 else 0

    @property
    def pos_hi(self) -> int:
        return (self.rank + 1) * self.shard_len if self.world_size > 1 else 2 ** 31 - 1


def local_context_lens(context_lens: torch.Tensor, shard: ShardInfo) -> torch.Tensor:
    """Keys of each request that fall into this rank's position range."""
    if shard.world_size == 1:
        return context_lens
    return (context_lens - shard.pos_lo).clamp(min=0, max=shard.shard_len).to(torch.int32)


class SparseDecodeStep:
    """Pre-allocated decode step for a fixed batch size.

    Per-step inputs (device tensors):
      q_idx   bf16 [B, 64, 128]   index queries        w      fp32 [B, 64] head weights
      q_lat   bf16 [B, H, 576]    absorbed MLA queries
    Persistent state (device tensors owned by the caller):
      k_cache uint8 paged FP8 index-key cache (this rank's pages), block_table int32 [B, pages]
      context_lens int32 [B] (global lengths), kv bf16 [rows, 576] latent cache (this rank's rows),
      kv_row_base int64 [B] row of each request's first local position.
    """

    def __init__(self, batch: int, max_local_ctx: int, *, page_size: int = 64, topk: int = 2048,
                 n_heads: int = 128, index_scale: float = 128 ** -0.5, attn_scale: float = 192 ** -0.5,
                 device: Optional[torch.device] = None, shard: Optional[ShardInfo] = None, backend=None,
                 sorted_topk: bool = False, wire: str = "bf16", ctx_dtype: torch.dtype = torch.float32,
                 combine: str = "auto", fused_select: bool = True, keep_logits: bool = True,
                 result: str = "replicated"):
        if backend is None:
            from . import kernels as backend  # the CUDA kernels; fails loudly without the library
        self.K = backend
        self.B, self.topk, self.H, self.P = batch, topk, n_heads, page_size
        self.index_scale, self.attn_scale = index_scale, attn_scale
        self.shard = shard or ShardInfo()
        self.sorted_topk = sorted_topk
        if wire not in ("bf16", "fp32"):
            raise ValueError("wire must be 'bf16' or 'fp32'")
        self.wire_mode = wire if hasattr(backend, "lse_prescale_norm") else "fp32"
        if combine not in ("auto", "peer", "nccl"):
            raise ValueError("combine must be 'auto', 'peer' or 'nccl'")
        if result not in ("replicated", "sharded"):
            raise ValueError("result must be 'replicated' (every rank ends with all rows) or 'sharded' (each rank "
                             "keeps the (item, head) rows of its slice: what a tensor-parallel output projection reads)")
        self.result = result
        dev = device if device is not None else torch.device("cuda")
        self.dev = dev
        f32, i32 = torch.float32, torch.int32
        n = self.shard.world_size
        self.max_cols = max_local_ctx
        self.logits = torch.empty(batch, max_local_ctx, dtype=f32, device=dev)
        self.q_fp8 = torch.empty(batch, 64, 128, dtype=torch.float8_e4m3fn, device=dev)
        self.weights = torch.empty(batch, 64, dtype=f32, device=dev)
        # candidate wire layout: [B, 2k] int32 = k global positions then k score bit patterns
        self.cand = torch.empty(batch, 2 * topk, dtype=i32, device=dev)
        self.pos_offset = torch.full((batch,), self.shard.pos_lo, dtype=i32, device=dev)
        # unsharded: the kernel writes the result in ctx_dtype (bf16 is what the reference op returns);
        # sharded: fp32 partials, merged by combine()
        self.ctx = torch.empty(batch, n_heads, 512, dtype=ctx_dtype if n == 1 else f32, device=dev)
        self.lse = torch.empty(batch, n_heads, dtype=f32, device=dev)
        self.q_pos = torch.empty(batch, dtype=i32, device=dev)
        # few long rows: spread the top-k of every row over several CTAs (global scratch, allocated once)
        self.topk_scratch = None
        if hasattr(backend, "topk_scratch") and batch <= 148 and max_local_ctx >= 16384:
            self.topk_scratch = backend.topk_scratch(batch, dev)
        # fused selection: the indexer's epilogue collects the top-k candidates itself (two launches, no
        # pass over the logits; they are still written, unless keep_logits=False, as the exact fallback)
        self.fused_scratch = None
        self.keep_logits = keep_logits
        if fused_select and hasattr(backend, "indexer_paged_fp8_topk") and topk <= 2048:
            self.fused_scratch = backend.fused_scratch(batch, dev)
        self.peer = None
        if combine == "peer" and not (n > 1 and dist.is_initialized()):
            raise ValueError("combine='peer' needs an initialised process group of more than one rank")
        if n > 1 and combine != "nccl" and dev.type == "cuda" and dist.is_initialized() and \
                getattr(backend, "__name__", "").endswith(".kernels"):
            self.cand_bytes = batch * 2 * topk * 4
            self.peer = self._open_peer_combine(batch * n_heads, dev, combine == "peer", self.cand_bytes * (1 + n))
        if self.peer is not None:
            # attention writes its normalised bf16 partial straight into the exchange buffer, the local
            # top-k its (position, score) candidates; the exchange kernels push both to the peers
            self.ctx = self.peer.ctx.view(batch, n_heads, 512)
            self.lse = self.peer.lse.view(batch, n_heads)
            extra = self.peer.extra_of(self.peer.rank)
            self.cand = extra[:self.cand_bytes].view(i32).view(batch, 2 * topk)
        # both exchanges folded into the compute kernels: the selection pushes its rows to the peers, the merge
        # waits for them and emits the owned keys, the attention kernel raises the "partial ready" flags
        self.peer_fused = self.peer is not None and self.fused_scratch is not None
        if n > 1:
            if self.peer is not None:     # receive area inside the exchange buffer: peers store into it
                self.cand_all = self.peer.extra_of(self.peer.rank)[self.cand_bytes:].view(i32).view(n, batch, 2 * topk)
            else:
                self.cand_all = torch.empty(n, batch, 2 * topk, dtype=i32, device=dev)
            self.merged = torch.empty(batch, topk, dtype=i32, device=dev)
            self.owned = torch.empty(batch, topk, dtype=i32, device=dev)
            self.owned_count = torch.empty(batch, dtype=i32, device=dev)
            self.lse_max = torch.empty(batch, n_heads, dtype=f32, device=dev)
            self.lse_out = torch.empty(batch, n_heads, dtype=f32, device=dev)
            if self.peer is not None:
                pass
            elif self.wire_mode == "bf16":
                self.lse_all = torch.empty(n, batch, n_heads, dtype=f32, device=dev)
                self.ctx_bf16 = torch.empty(batch, n_heads, 512, dtype=torch.bfloat16, device=dev)
            else:
                self.wire_rows = torch.empty(batch * n_heads, backend.WIRE_ROW, dtype=f32, device=dev)
                self.ctx_out = torch.empty(batch, n_heads, 512, dtype=f32, device=dev)

    def _open_peer_combine(self, n_rows: int, dev, required: bool, extra_bytes: int):
        """Map the exchange buffers of all ranks (they must share a node).  Every rank learns
        whether all succeeded, so that the group takes the same path."""
        from .peer import PeerLseCombine
        peer, err = None, None
        try:
            peer = PeerLseCombine(n_rows, dev, self.shard.group, extra_bytes=extra_bytes)
        except Exception as e:                                   # noqa: BLE001 - reported below
            err = e
        ok = torch.tensor([0 if peer is None else 1], dtype=torch.int32, device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=self.shard.group)
        if int(ok.item()) == 1:
            return peer
        if peer is not None:
            peer.close()
        if required:
            raise RuntimeError(f"peer-memory combine is not available on every rank: {err}")
        import warnings
        warnings.warn(f"peer-memory combine unavailable ({err}); merging through NCCL")
        return None

    # ------------------------------------------------------------------ stages
    def select(self, q_idx, w, k_cache, context_lens_local, block_table) -> torch.Tensor:
        """Indexer + top-k on this rank's keys; returns int32 [B, k] global positions."""
        K = self.K
        K.quant_q_fold_weights(q_idx, w, self.index_scale, q_fp8=self.q_fp8, weights=self.weights)
        idx = self.cand[:, : self.topk]
        val = self.cand[:, self.topk:].view(torch.float32)
        offset = self.pos_offset if self.shard.world_size > 1 else None
        if self.fused_scratch is not None:
            push = None
            if self.peer_fused:           # receive area: right after this rank's own candidates in the extra area
                push = (self.peer.link(1), self.peer.off_extra + self.cand_bytes)
            K.indexer_paged_fp8_topk(self.q_fp8, self.weights, k_cache, self.P, context_lens_local, block_table,
                                     self.topk, self.fused_scratch, max_cols=self.max_cols, logits=self.logits,
                                     keep_logits=self.keep_logits, row_pos_offset=offset, sorted=self.sorted_topk,
                                     out=idx, out_values=val, push=push)
            return idx
        K.indexer_paged_fp8_logits(self.q_fp8, self.weights, k_cache, self.P, context_lens_local, block_table,
                                   max_cols=self.max_cols, out=self.logits)
        if self.topk_scratch is not None:
            K.topk_select_split(self.logits, self.topk, self.topk_scratch, col_end=context_lens_local,
                                sorted=self.sorted_topk, row_pos_offset=offset, out=idx, out_values=val)
        else:
            K.topk_select(self.logits, self.topk, col_end=context_lens_local, sorted=self.sorted_topk,
                          row_pos_offset=offset, out=idx, out_values=val)
        return idx

    def merge_candidates(self) -> torch.Tensor:
        """All-gather the per-rank candidates and select the global top-k (identical on every rank)."""
        n, k = self.shard.world_size, self.topk
        if self.peer_fused:
            # the selections pushed their rows already: wait for the peers' flags inside the merge kernel,
            # which also compacts the winners this rank owns
            self.K.topk_merge_owned(self.cand_all, k, self.shard.pos_lo, self.shard.pos_hi, out=self.merged,
                                    owned=self.owned, owned_count=self.owned_count, sorted=self.sorted_topk,
                                    link=self.peer.link(1))
            return self.merged
        if self.peer is not None:
            # one kernel: this rank's candidates are stored into its slot of every rank's receive area
            # (posted NVLink stores, same layout as the NCCL all-gather delivers); it ends when all
            # peers' slots have landed here
            self.peer.push_extra(self.cand_bytes, slot=1)
        else:
            dist.all_gather_into_tensor(self.cand_all.view(-1), self.cand.view(-1), group=self.shard.group)
        flat = self.cand_all.view(-1)
        scores = flat[k:].view(torch.float32)        # segment r, row b starts at r*B*2k + b*2k + k
        pos = flat                                   # positions start at r*B*2k + b*2k
        self.K.topk_select(scores.view(1, -1), k, sorted=self.sorted_topk, pos_map=pos.view(1, -1),
                           out=self.merged, n_cols=n * k, row_stride=2 * k, seg_cols=k,
                           seg_stride=self.B * 2 * k, n_rows=self.B, pos_map_stride=2 * k)
        return self.merged

    def attend(self, q_lat, kv, kv_row_base, indices, q_pos, q_pos_bias: int = 0,
               signal: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
        """Attention over the selected keys this rank owns (all of them when unsharded).  Keys beyond
        q_pos + q_pos_bias are masked (context lengths with a bias of -1 save a subtraction kernel).
        signal=False: do not tell the peers that the partial is ready (combine() then does, as when the
        exchanges are separate kernels)."""
        count = None
        self._signalled = False
        if self.peer_fused and indices is self.merged:
            self._signalled = signal
            return self.K.sparse_mla_decode(q_lat, kv, self.owned, self.attn_scale, kv_row_base=kv_row_base, q_pos=q_pos,
                                            pos_lo=self.shard.pos_lo, pos_hi=self.shard.pos_hi,
                                            n_idx_item=self.owned_count, ctx=self.ctx, lse=self.lse,
                                            q_pos_bias=q_pos_bias,
                                            signal=(self.peer.link(0), self.peer.ticket) if signal else None)
        if self.shard.world_size > 1 and hasattr(self.K, "compact_owned"):
            # only about 1/N of the selection lives here: compact it so the kernel walks just those
            indices, count = self.K.compact_owned(indices, self.shard.pos_lo, self.shard.pos_hi, self.owned,
                                                  self.owned_count)
        return self.K.sparse_mla_decode(q_lat, kv, indices, self.attn_scale, kv_row_base=kv_row_base, q_pos=q_pos,
                                        pos_lo=self.shard.pos_lo, pos_hi=self.shard.pos_hi, n_idx_item=count,
                                        ctx=self.ctx, lse=self.lse, q_pos_bias=q_pos_bias)

    def combine(self) -> Tuple[torch.Tensor, torch.Tensor]:
        """Merge the per-rank (ctx, lse) partials; every rank ends with the full result."""
        K, g = self.K, self.shard.group
        if self.peer is not None:
            # one kernel: flags, peer loads of all partials of the rows this rank owns, merged rows
            # stored to every rank
            out, lse_out = self.peer.run(pre_signalled=getattr(self, "_signalled", False),
                                         local_only=self.result == "sharded")
            return out.view(self.B, self.H, 512), lse_out.view(self.B, self.H)
        if self.wire_mode == "bf16":
            # gather the lse of every rank (4 B per row and rank): each rank then knows the common
            # maximum and the exact denominator and sends its normalised bf16 share; the summed
            # rows are the result
            dist.all_gather_into_tensor(self.lse_all.view(-1), self.lse.view(-1), group=g)
            K.lse_prescale_norm(self.ctx, self.lse_all, self.shard.rank, self.ctx_bf16, self.lse_out)
            dist.all_reduce(self.ctx_bf16, op=dist.ReduceOp.SUM, group=g)
            return self.ctx_bf16, self.lse_out
        self.lse_max.copy_(self.lse)
        dist.all_reduce(self.lse_max, op=dist.ReduceOp.MAX, group=g)
        K.lse_prescale(self.ctx, self.lse, self.lse_max, self.wire_rows)
        dist.all_reduce(self.wire_rows, op=dist.ReduceOp.SUM, group=g)
        return K.lse_finalize(self.wire_rows, self.lse_max, self.ctx_out, self.lse_out)

    # ------------------------------------------------------------------ whole step
    def run(self, q_idx, w, q_lat, k_cache, context_lens, block_table, kv, kv_row_base,
            context_lens_local: Optional[torch.Tensor] = None):
        """Returns (indices int32 [B,k] global positions, ctx [B,H,512], lse fp32 [B,H]); ctx is
        ctx_dtype when unsharded, bf16 / fp32 after a sharded combine with the bf16 / fp32 wire."""
        if context_lens_local is None:
            context_lens_local = local_context_lens(context_lens, self.shard)
        idx = self.select(q_idx, w, k_cache, context_lens_local, block_table)
        if self.shard.world_size > 1:
            idx = self.merge_candidates()
        ctx, lse = self.attend(q_lat, kv, kv_row_base, idx, context_lens, q_pos_bias=-1)
        if self.shard.world_size > 1:
            ctx, lse = self.combine()
        return idx, ctx, lse


def input_layout(batch: int, n_heads: int) -> dict:
    """Byte offsets of (q_idx bf16 [B,64,128], w fp32 [B,64], q_lat bf16 [B,H,576]) inside one packed buffer
    (each part starts on a 256-byte boundary)."""
    sizes = (batch * 64 * 128 * 2, batch * 64 * 4, batch * n_heads * 576 * 2)
    offs, o = [], 0
    for n in sizes:
        offs.append(o)
        o += (n + 255) // 256 * 256
    return {"offsets": tuple(offs), "sizes": sizes, "bytes": o}


def unpack_inputs(buf: torch.Tensor, batch: int, n_heads: int):
    """(q_idx, w, q_lat) as views of a packed uint8 buffer (input_layout)."""
    lay = input_layout(batch, n_heads)
    (o0, o1, o2), (n0, n1, n2) = lay["offsets"], lay["sizes"]
    return (buf[o0:o0 + n0].view(torch.bfloat16).view(batch, 64, 128),
            buf[o1:o1 + n1].view(torch.float32).view(batch, 64),
            buf[o2:o2 + n2].view(torch.bfloat16).view(batch, n_heads, 576))


def pack_inputs(q_idx: torch.Tensor, w: torch.Tensor, q_lat: torch.Tensor, out: torch.Tensor = None) -> torch.Tensor:
    """Copy the three inputs into one uint8 buffer (allocated on q_idx's device when not given)."""
    B, H = q_idx.shape[0], q_lat.shape[1]
    lay = input_layout(B, H)
    if out is None:
        out = torch.empty(lay["bytes"], dtype=torch.uint8, device=q_idx.device)
    for dst, src in zip(unpack_inputs(out, B, H), (q_idx, w, q_lat)):
        dst.copy_(src)
    return out


class GraphedDecodeStep:
    """The whole step captured once into a CUDA graph and replayed: per-step host work drops to
    one graph launch (the kernels' host calls, tensor-map encodes and NCCL enqueues are recorded
    at capture time).  Inputs are copied into static buffers before each replay; outputs are the
    step's own pre-allocated buffers.  Capture after at least one eager run (so that lazy
    initialisation, e.g. NCCL communicators, is done) and never while another capture is active."""

    def __init__(self, step: SparseDecodeStep, k_cache, context_lens, block_table, kv, kv_row_base,
                 context_lens_local=None):
        self.step = step
        dev = step.dev
        B, H = step.B, step.H
        # the three inputs are views of one byte buffer, so that a serving loop can stage a step's inputs in one
        # pinned arena and bring them in with one copy (replay_packed)
        self.layout = input_layout(B, H)
        self.inputs = torch.empty(self.layout["bytes"], dtype=torch.uint8, device=dev)
        self.q_idx, self.w, self.q_lat = unpack_inputs(self.inputs, B, H)
        self._state = (k_cache, context_lens, block_table, kv, kv_row_base, context_lens_local)
        self.graph = None
        self.out = None

    def capture(self):
        k_cache, context_lens, block_table, kv, kv_row_base, local = self._state
        if local is None:
            local = local_context_lens(context_lens, self.step.shard)
            self._state = (k_cache, context_lens, block_table, kv, kv_row_base, local)
        side = torch.cuda.Stream(device=self.step.dev)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):            # warm-up on the capture stream
            self.step.run(self.q_idx, self.w, self.q_lat, k_cache, context_lens, block_table, kv, kv_row_base, local)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.out = self.step.run(self.q_idx, self.w, self.q_lat, k_cache, context_lens, block_table, kv,
                                     kv_row_base, local)
        return self

    def replay_packed(self, packed: torch.Tensor):
        """One copy of a packed input buffer (pack_inputs layout; device or pinned host), then replay."""
        self.inputs.copy_(packed, non_blocking=True)
        self.graph.replay()
        return self.out

    def replay(self, q_idx=None, w=None, q_lat=None):
        """Copy the given inputs (device or pinned host tensors) into the static buffers and replay."""
        if q_idx is not None:
            self.q_idx.copy_(q_idx, non_blocking=True)
            self.w.copy_(w, non_blocking=True)
            self.q_lat.copy_(q_lat, non_blocking=True)
        self.graph.replay()
        return self.out


class PipelinedDecode:
    """A serving loop over host buffers without device-side staging copies: several captured steps, each with its
    own input and result buffers, are used in turn, so that the host-to-device copy of step i+1 lands straight
    in the static input buffer of its graph while the kernels of step i run, and the device-to-host copy of step
    i-1 reads the result buffers of its graph.  (With a single graph the inputs and results have to pass through
    per-slot device buffers: three device-to-device copies per step.)  Single-GPU steps only: the captured steps
    of a key-sharded run share one exchange buffer and its step counters.

        pipe = PipelinedDecode([GraphedDecodeStep(step_a, ...).capture(), GraphedDecodeStep(step_b, ...).capture()])
        slot = pipe.submit(packed_pinned)       # inputs in pack_inputs layout, page-locked host memory
        idx, ctx = pipe.result(slot)            # page-locked host tensors, valid until the slot is submitted again
    """

    def __init__(self, graphs: Sequence["GraphedDecodeStep"]):
        if len(graphs) < 2:
            raise ValueError("PipelinedDecode needs at least two captured steps")
        for g in graphs:
            if g.graph is None or g.step.shard.world_size != 1:
                raise ValueError("PipelinedDecode takes captured single-GPU steps")
        self.graphs = list(graphs)
        dev = graphs[0].step.dev
        n = len(graphs)
        self.s_in, self.s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
        self.ev_in = [torch.cuda.Event() for _ in range(n)]
        self.ev_done = [torch.cuda.Event() for _ in range(n)]
        self.ev_out = [torch.cuda.Event() for _ in range(n)]
        self.started = [False] * n
        self.host_out = [(torch.empty(g.out[0].shape, dtype=g.out[0].dtype).pin_memory(),
                          torch.empty(g.out[1].shape, dtype=g.out[1].dtype).pin_memory()) for g in graphs]
        self.count = 0

    def submit(self, packed_host: torch.Tensor) -> int:
        """Enqueue one step on the next slot; returns the slot.  Blocks only until that slot's previous result
        has reached the host (its graph's buffers are free then)."""
        sl = self.count % len(self.graphs)
        self.count += 1
        g = self.graphs[sl]
        main = torch.cuda.current_stream()
        if self.started[sl]:
            self.ev_out[sl].synchronize()
        with torch.cuda.stream(self.s_in):
            g.inputs.copy_(packed_host, non_blocking=True)
            self.ev_in[sl].record(self.s_in)
        main.wait_event(self.ev_in[sl])
        g.graph.replay()
        self.ev_done[sl].record(main)
        self.s_out.wait_event(self.ev_done[sl])
        with torch.cuda.stream(self.s_out):
            self.host_out[sl][0].copy_(g.out[0], non_blocking=True)
            self.host_out[sl][1].copy_(g.out[1], non_blocking=True)
            self.ev_out[sl].record(self.s_out)
        self.started[sl] = True
        return sl

    def result(self, slot: int):
        """(indices, ctx) of the last step submitted on `slot`, on the host."""
        self.ev_out[slot].synchronize()
        return self.host_out[slot]
