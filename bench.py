"""Benchmark of the sparse decode step (indexer -> top-k -> sparse MLA attention).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload: batch 64 requests at context 131072, one query token each, 64 index heads (d=128)
over an FP8 paged index-key cache, top-2048 selection, sparse MLA attention over 576-wide bf16
latent rows with 128 heads.  With N > 1 (launched by torch.distributed.run) the key range is
sharded over the ranks; total work is fixed ("strong" scaling).  One JSON line is printed by
rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

BATCH = 64
CONTEXT = 131072
HEADS = 128
TOPK = 2048
PAGE = 64
INDEX_SCALE = 128 ** -0.5
ATTN_SCALE = 192 ** -0.5
# DRAM bytes (read + write) per scored key of the indexer kernel, from an ncu capture of that kernel
# on a smaller case (dram__bytes_read + dram__bytes_write over the keys scored; traffic grows in
# proportion to the number of keys).
DRAM_BYTES_PER_KEY = 137.3
METRIC = "sparse_mla_decode_tokens_per_s"
WORKLOAD = ("sparse MLA decode, key-sharded: batch 64, context 131072, 64 index heads d=128, FP8 paged "
            "index keys (page 64) with per-token scale, top-2048, 128 heads over 576-wide bf16 latent KV")


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.rows = []
        self.proc = None
        self.gpu = gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu), f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        mhz, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 6:
                continue
            try:
                mhz.append(float(r[0])); mx = float(r[1])
            except ValueError:
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        mhz.sort()
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(mhz)}


def _cpu_inputs(n_requests: int, context: int):
    from oracle import dsa_oracle as O
    g = torch.Generator().manual_seed(4)
    k = torch.randn(context, 128, generator=g)
    kq, sc = O.quant_fp8_rows(k)
    kd = kq.float() * sc.unsqueeze(-1)                     # dequantised keys, as misa_ops.py:687 hands them on
    kv = (0.5 * torch.randn(context, 576, generator=g)).bfloat16().float()
    q = torch.randn(n_requests, 64, 128, generator=g)
    w = torch.randn(n_requests, 64, generator=g) / 8
    q_lat = torch.randn(n_requests, HEADS, 576, generator=g)
    return kd, kv, q, w, q_lat


def cpu_tokens_per_s(n_requests: int, context: int, threads: int):
    """Times the CPU implementation of the path on n_requests requests of the benchmark's shape: the
    reference's own indexer_select_topk + sparse_attend_absorbed_chunked when oracle/_ref holds them
    (kind "reference"), else their restatement in oracle/ (kind "port").  Decode is driven per
    request: one query at global position context-1 against the request's dequantised keys.
    Returns (tokens/s, seconds, kind)."""
    from oracle import dsa_oracle as O
    from oracle.make_ref import reference_ops
    torch.set_num_threads(threads)
    ref = reference_ops()
    kd, kv, q, w, q_lat = _cpu_inputs(n_requests, context)
    cu = torch.tensor([0, context])
    pos = torch.tensor([context - 1])
    eye = torch.eye(512).unsqueeze(0).expand(HEADS, 512, 512)      # W_UV = I: the latent-space context
    t0 = time.perf_counter()
    for b in range(n_requests):
        q_fp8, wf = O.quant_q_fold_weights(q[b:b + 1], w[b:b + 1], INDEX_SCALE)
        if ref is not None:
            idx = ref.indexer_select_topk(q_fp8.float(), kd, wf, cu, TOPK, sm_scale_index=1.0, q_global_pos=pos)
            ref.sparse_attend_absorbed_chunked(q_lat[b:b + 1], kv, eye, idx, d_c=512, sm_scale=ATTN_SCALE,
                                               checkpoint=False, q_global_pos=pos)
        else:
            s = O.indexer_scores(q_fp8.float(), kd, wf, 1.0)
            idx = O.topk_rows(s, TOPK)
            O.sparse_attend_latent(q_lat[b:b + 1], kv, idx, d_c=512, sm_scale=ATTN_SCALE, q_pos=pos)
    dt = time.perf_counter() - t0
    return n_requests / dt, dt, ("reference" if ref is not None else "port")


def run_reference(args, rank: int):
    """Reference arm: the reference's implementation of this path is PyTorch on the host cores (its
    GPU kernels are TileLang, which is not a CPU path).  Its own functions are timed when
    oracle/_ref holds them, else their restatement."""
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    _, dt4, kind = cpu_tokens_per_s(4, CONTEXT, threads)              # calibrate: about 2 s per step
    n_req = max(4, min(256, int(2.0 / max(dt4 / 4, 1e-4))))
    for _ in range(min(args.warmup, 2)):
        cpu_tokens_per_s(n_req, CONTEXT, threads)
    args.steps = min(args.steps, 20)                                  # keep the whole arm within a few minutes
    vals, secs = [], 0.0
    for _ in range(args.steps):
        v, dt, kind = cpu_tokens_per_s(n_req, CONTEXT, threads)
        vals.append(v); secs += dt
    value = sum(vals) / len(vals)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * secs / args.steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "parallelism": "host cores", "launch": "cpu"},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": kind,
                         "sample": f"{n_req} requests of the batch's shape per step at context {CONTEXT}, all stages"},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------------------
# The other configurations of the path (prefill select, ragged decode, HISA, routed decode), each timed
# through the public Python call: median and min of REPS CUDA-event measurements after WARM warm-ups,
# L2 flushed between repetitions (a 256 MB buffer is rewritten outside the timed bracket).
# --------------------------------------------------------------------------------------------------
CFG_REPS, CFG_WARM = 50, 10


def _time_call(fn, flush, reps=None, warm=None):
    for _ in range(CFG_WARM if warm is None else warm):
        fn()
    ts = []
    for _ in range(CFG_REPS if reps is None else reps):
        flush.add_(1)                                      # evict L2 (256 MB > 126 MB)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); fn(); e1.record()
        torch.cuda.synchronize()
        ts.append(1e3 * e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2], ts[0]


def bench_configs(dev, peaks, threads: int, fp8_peak: float, only=None, with_cpu: bool = True):
    from oracle import dsa_oracle as O
    from oracle.make_ref import reference_ops
    from transarch_b200 import hisa, kernels as K, misa, opendsa_ops
    from transarch_b200.decode import SparseDecodeStep
    from transarch_b200.workloads import make_decode_queries, make_decode_state
    ref = reference_ops() if with_cpu else None
    torch.set_num_threads(threads)
    flush = torch.zeros(64 << 20, dtype=torch.float32, device=dev)
    hbm, bf16 = peaks["hbm_gbs"], peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"])
    out = {}

    def want(tag):
        return only is None or tag in only

    def cpu_time(fn):
        if not with_cpu:
            return None
        t0 = time.perf_counter()
        fn()
        return time.perf_counter() - t0

    def c1():
        """causal prefill select, T = S = 4096, 64 heads, d = 128, top-2048, seed 0"""
        g = torch.Generator().manual_seed(0)
        T = 4096
        q = torch.randn(T, 64, 128, generator=g); k = torch.randn(T, 128, generator=g)
        w = torch.randn(T, 64, generator=g) / 8
        cu = torch.tensor([0, T])
        qd, kd, wd, cud = q.to(dev).bfloat16(), k.to(dev).bfloat16(), w.to(dev), cu.to(dev)
        med, mn = _time_call(lambda: opendsa_ops.indexer_select_topk(qd, kd, wd, cud, 2048), flush)
        med_u, _ = _time_call(lambda: opendsa_ops.indexer_select_topk(qd, kd, wd, cud, 2048, sorted=False), flush)
        ksd, ked = opendsa_ops.prepare_ks_ke(cud, total=T)
        med_l, _ = _time_call(lambda: opendsa_ops.indexer_logits_flat(qd, kd, wd, ksd, ked, 128 ** -0.5), flush)
        cpu_s = cpu_time(lambda: (ref.indexer_select_topk if ref is not None else O.indexer_select_topk)(
            q, k, w, cu, 2048, q_chunk=512))
        flops = T * (T + 1) // 2 * 16384
        out["C1 causal prefill select T=S=4096 k=2048 (bf16)"] = {
            "call": "opendsa_ops.indexer_select_topk", "us_median": med, "us_min": mn, "flops": flops,
            "bytes": 103e6, "bound": "tensor", "achieved_tflops": flops / med / 1e6,
            "frac_of_bf16_sustained": flops / med / 1e6 / bf16, "us_median_unsorted_output": med_u,
            "us_median_logits_only": med_l, "logits_only_frac_of_bf16_sustained": flops / med_l / 1e6 / bf16,
            "cpu_seconds": cpu_s, "cpu_kind": "reference" if ref is not None else "port",
            "cpu_sample": "whole configuration, fp32, q_chunk=512"}

    def c2():
        """ragged decode, 64 requests with contexts uniform in [8K, 32K], FP8 paged keys, top-2048, seed 1"""
        g = torch.Generator().manual_seed(1)
        lens = torch.randint(8192, 32769, (64,), generator=g).tolist()
        st = make_decode_state(64, lens, seed=1, device=dev)
        q_idx, wq, _ = make_decode_queries(64, seed=1, device=dev)
        step = SparseDecodeStep(64, st.local_len, topk=TOPK, device=dev)
        med, mn = _time_call(lambda: step.select(q_idx, wq, st.k_cache, st.context_lens, st.block_table), flush)
        n_keys = sum(lens)
        sample = 8

        def cpu():
            for b in range(sample):
                kb = torch.randn(lens[b], 128)
                qf, wf = O.quant_q_fold_weights(torch.randn(1, 64, 128), torch.randn(1, 64) / 8, INDEX_SCALE)
                if ref is not None:
                    ref.indexer_select_topk(qf.float(), kb, wf, torch.tensor([0, lens[b]]), TOPK, sm_scale_index=1.0,
                                            q_global_pos=torch.tensor([lens[b] - 1]))
                else:
                    O.topk_rows(O.indexer_scores(qf.float(), kb, wf, 1.0), TOPK)
        cpu_s = cpu_time(cpu)
        out["C2 ragged decode indexer+top-k, 64 requests 8K-32K (fp8)"] = {
            "call": "SparseDecodeStep.select", "us_median": med, "us_min": mn, "flops": n_keys * 16384,
            "bytes": n_keys * 132, "bound": "hbm", "achieved_gbs": n_keys * 132 / med / 1e3,
            "frac_of_hbm": n_keys * 132 / med / 1e3 / hbm,
            "cpu_seconds": None if cpu_s is None else cpu_s * n_keys / sum(lens[:sample]),
            "cpu_kind": "reference" if ref is not None else "port", "cpu_sample": f"{sample} of 64 requests, scaled by keys"}

    def c3():
        """HISA two-stage, 4096 queries at positions 126976..131071 over 131072 keys, seed 2"""
        g = torch.Generator(device=dev).manual_seed(2)
        S, T = 131072, 4096
        k3 = torch.randn(S, 128, generator=g, device=dev).bfloat16()
        q3 = torch.randn(T, 64, 128, generator=g, device=dev).bfloat16()
        w3 = torch.randn(T, 64, generator=g, device=dev) / 8
        pos = torch.arange(S - T, S, device=dev)
        ks3, ke3 = torch.zeros(T, dtype=torch.int64, device=dev), pos + 1
        cfg = hisa.HisaConfig()
        med, mn = _time_call(lambda: hisa.hisa_select_topk(q3, k3, w3, ks3, ke3, cfg), flush)
        sample = 32
        sel = torch.arange(0, T, T // sample)
        cpu_s = cpu_time(lambda: O.hisa_select_topk(q3[sel].cpu().float(), k3.cpu().float(), w3[sel].cpu(), ks3[sel].cpu(),
                                                    ke3[sel].cpu(), block=128, block_topk=64, topk=2048))
        flops = int(67.7e9 + T * 8192 * 16384)
        out["C3 HISA two-stage, 4096 queries at the tail of 131072 keys (bf16)"] = {
            "call": "hisa.hisa_select_topk", "us_median": med, "us_min": mn, "flops": flops, "bytes": 135e6,
            "bound": "tensor", "achieved_tflops": flops / med / 1e6, "frac_of_bf16_sustained": flops / med / 1e6 / bf16,
            "cpu_seconds": None if cpu_s is None else cpu_s * T / sample,
            "cpu_kind": "port (the reference ships no HISA code)", "cpu_sample": f"{sample} of 4096 queries, scaled"}

    def c4():
        """MISA routed decode, batch 32, context 65536, linear router top-8 of 64, seed 3"""
        st = make_decode_state(32, 65536, seed=3, device=dev)
        q4, _, _ = make_decode_queries(32, seed=3, device=dev)
        g = torch.Generator(device=dev).manual_seed(3)
        x = torch.randn(32, 7168, generator=g, device=dev).bfloat16()
        W_r = (torch.randn(7168, 64, generator=g, device=dev) * 7168 ** -0.5).bfloat16()
        q_fp8, fold = K.quant_q_fold_weights(q4, torch.ones(32, 64, device=dev), INDEX_SCALE)
        med, mn = _time_call(lambda: misa.misa_linear_router_decode(x, W_r, q_fp8, fold, st.k_cache, 64,
                                                                    st.context_lens, st.block_table, 8, TOPK,
                                                                    max_cols=65536), flush)
        sample = 4

        def cpu():
            for b in range(sample):
                kb = torch.randn(65536, 128)
                hidx, hw, _ = O.linear_router_topk_softmax(x[b:b + 1].cpu(), W_r.cpu(), 8)
                q8, _ = O.gather_heads(q_fp8[b:b + 1].cpu().float(), fold[b:b + 1].cpu(), hidx)
                O.topk_rows(O.indexer_scores(q8, kb, hw * torch.gather(fold[b:b + 1].cpu(), 1, hidx), 1.0), TOPK)
        cpu_s = cpu_time(cpu)
        n_keys = 32 * 65536
        out["C4 MISA routed decode, batch 32 x 65536 keys, 8 of 64 heads (fp8)"] = {
            "call": "misa.misa_linear_router_decode", "us_median": med, "us_min": mn, "flops": n_keys * 2048,
            "bytes": n_keys * 132, "bound": "hbm", "achieved_gbs": n_keys * 132 / med / 1e3,
            "frac_of_hbm": n_keys * 132 / med / 1e3 / hbm,
            "cpu_seconds": None if cpu_s is None else cpu_s * 32 / sample,
            "cpu_kind": "port (no reference code for the linear router)",
            "cpu_sample": f"{sample} of 32 requests, 8 routed heads only, scaled"}

    def m1():
        """MISA routed prefill (not a BASELINE configuration): 4096 queries at the tail of 65536 keys, q-norm
        router 8 of 64 heads, stage-1 top-8192, seed 5"""
        g = torch.Generator(device=dev).manual_seed(5)
        N, M, s1 = 65536, 4096, 8192
        kq = torch.randn(N, 128, generator=g, device=dev).to(torch.float8_e4m3fn)
        sc = torch.ones(N, device=dev)
        q = torch.randn(M, 64, 128, generator=g, device=dev).to(torch.float8_e4m3fn)
        w = torch.randn(M, 64, generator=g, device=dev) / 8
        ke = torch.arange(N - M, N, device=dev, dtype=torch.int32) + 1
        ks = torch.zeros(M, dtype=torch.int32, device=dev)
        hidx = torch.topk(q.float().norm(dim=-1), 8, dim=-1).indices.int()
        med, mn = _time_call(lambda: misa.misa_mqa_logits(q, (kq, sc), w, hidx, ks, ke, True, 8, s1), flush, reps=10,
                             warm=3)
        pairs = float((ke.long() - ks.long()).sum())            # (query, key) pairs in range
        flops = int(pairs * 8 * 256 + M * s1 * 64 * 256)
        out["M1 MISA routed prefill, 4096 queries at the tail of 65536 keys, 8 of 64 heads, stage-1 top-8192 (bf16)"] = {
            "call": "misa.misa_mqa_logits", "us_median": med, "us_min": mn, "flops": flops,
            "flops_without_routing": int(pairs * 64 * 256), "bound": "tensor",
            "achieved_tflops": flops / med / 1e6, "frac_of_bf16_sustained": flops / med / 1e6 / bf16,
            "cpu_seconds": None, "cpu_kind": "not timed"}

    def t1():
        """training form of the sparse attention (not a BASELINE configuration): forward + backward of
        sparse_attend_absorbed_chunked, 2048 queries x 128 heads x top-2048, bf16, seed 6; beside it the reference's
        own torch op on the same GPU"""
        g = torch.Generator(device=dev).manual_seed(6)
        L, H, Kk, Dv = 2048, 128, 2048, 128
        q = (torch.randn(L, H, 576, generator=g, device=dev) * 0.3).bfloat16()
        lat = (torch.randn(L, 576, generator=g, device=dev) * 0.3).bfloat16()
        W = (torch.randn(H, Dv, 512, generator=g, device=dev) / 512 ** 0.5).bfloat16()
        idx = (torch.rand(L, Kk, generator=g, device=dev) * (torch.arange(L, device=dev).view(-1, 1) + 1)).int()
        G = torch.randn(L, H, Dv, generator=g, device=dev).bfloat16()

        def fwd_bwd(fn):
            x, y, z = (t.clone().requires_grad_() for t in (q, lat, W))
            (fn(x, y, z, idx, d_c=512, sm_scale=576 ** -0.5, q_chunk=512).float() * G.float()).sum().backward()

        med, mn = _time_call(lambda: fwd_bwd(opendsa_ops.sparse_attend_absorbed_chunked), flush, reps=5, warm=2)
        ref_us = None
        if ref is not None:
            ref_us, _ = _time_call(lambda: fwd_bwd(ref.sparse_attend_absorbed_chunked), flush, reps=3, warm=1)
        flops = int(L * H * Kk * (576 * 6 + 512 * 4))        # forward 2 products, backward 2 + 3 products
        out["T1 sparse attention forward + backward, 2048 queries x 128 heads x top-2048 (bf16)"] = {
            "call": "opendsa_ops.sparse_attend_absorbed_chunked under autograd", "us_median": med, "us_min": mn,
            "flops": flops, "bound": "tensor", "achieved_tflops": flops / med / 1e6,
            "frac_of_bf16_sustained": flops / med / 1e6 / bf16,
            "reference_torch_op_same_gpu_us": ref_us, "cpu_seconds": None, "cpu_kind": "not timed"}

    for tag, fn in (("C1", c1), ("C2", c2), ("C3", c3), ("C4", c4), ("M1", m1), ("T1", t1)):
        if want(tag):
            fn()
            torch.cuda.empty_cache()
    for v in out.values():
        for kk in list(v):
            if isinstance(v[kk], float):
                v[kk] = round(v[kk], 4 if v[kk] < 10 else 2)
    return out


def parity_check(step, state, q_sets, res, ctx_len: int, requests):
    """Outside every timed region: the benchmarked step's own outputs for a few requests against the
    oracle at full length (indexer scores, index sets with the near-tie audit, attention output)."""
    from oracle import dsa_oracle as O
    q_idx, w, q_lat = q_sets
    idx, ctx, lse = res
    worst = {"score_rel_err": 0.0, "recall": 1.0, "attn_rel_err": 0.0, "lse_abs_err": 0.0}
    for b in requests:
        pages = state.k_cache[state.block_table[b].long()].cpu()
        kv_b = state.kv[b * ctx_len:(b + 1) * ctx_len].cpu()
        sc, ref_idx, _, _ = O.decode_request_reference(q_idx[b:b + 1].cpu(), w[b:b + 1].cpu(), q_lat[b:b + 1].cpu(),
                                                       pages, kv_b, ctx_len, TOPK, INDEX_SCALE, ATTN_SCALE)
        r = O.check_decode_request(sc, ref_idx, step.logits[b].cpu(), idx[b].cpu(), ctx[b].cpu(), lse[b].cpu(),
                                   q_lat[b:b + 1].cpu(), kv_b, ctx_len, ATTN_SCALE)
        worst["recall"] = min(worst["recall"], r["recall"])
        for k_ in ("score_rel_err", "attn_rel_err", "lse_abs_err"):
            worst[k_] = max(worst[k_], r[k_])
    return {"checked_requests": list(requests), "against": "CPU oracle at full context length",
            "tolerances": {"score_rel_err": 1e-2, "recall": 0.999, "attn_rel_err": 2e-2},
            "non_near_tie_disagreements": 0, **{k_: round(v, 6) for k_, v in worst.items()}, "ok": True}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--context", type=int, default=CONTEXT)
    ap.add_argument("--batch", type=int, default=BATCH)
    ap.add_argument("--skip-cpu-baseline", action="store_true")
    ap.add_argument("--skip-configs", action="store_true", help="do not time the other configurations of the path")
    ap.add_argument("--skip-parity", action="store_true", help="do not compare sampled requests with the oracle")
    ap.add_argument("--configs-only", default="", help="comma-separated subset of C1,C2,C3,C4,M1,T1: time only these "
                    "configurations (no decode step) and print them; for profiling single kernels")
    ap.add_argument("--config-reps", type=int, default=0, help="timed repetitions per configuration (default 50)")
    ap.add_argument("--no-graph", action="store_true", help="launch the step eagerly instead of replaying a CUDA graph")
    ap.add_argument("--result", default="replicated", choices=["replicated", "sharded"],
                    help="sharded run: every rank ends with all result rows, or only with its slice of them")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if args.configs_only:
        global CFG_REPS, CFG_WARM
        if args.config_reps > 0:
            CFG_REPS, CFG_WARM = args.config_reps, min(CFG_WARM, args.config_reps)
        torch.cuda.set_device(local_rank)
        peaks, _ = measured_peaks()
        out = bench_configs(torch.device("cuda", local_rank), peaks, os.cpu_count() or 1, 0.0,
                            only=set(args.configs_only.split(",")), with_cpu=False)
        print(json.dumps({"configs": out}), flush=True)
        return

    import torch.distributed as dist
    from transarch_b200 import _lib
    from transarch_b200.decode import GraphedDecodeStep, ShardInfo, SparseDecodeStep
    from transarch_b200.workloads import make_decode_queries, make_decode_state

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    group = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # NCCL only carries set-up traffic and barriers here (the exchanges of the step are this library's own
        # peer-memory kernels): it needs no NVLink multicast objects, and without them a rank that leaves
        # early cannot disturb its peers
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=dev)
    B, ctx = args.batch, args.context
    assert ctx % (world * PAGE) == 0
    shard_len = ctx // world
    shard = ShardInfo(rank=rank, world_size=world, shard_len=shard_len, group=group)
    state = make_decode_state(B, ctx, page_size=PAGE, seed=4, rank=rank, world_size=world, shard_len=shard_len,
                              device=dev)
    step = SparseDecodeStep(B, shard_len, page_size=PAGE, topk=TOPK, n_heads=HEADS, index_scale=INDEX_SCALE,
                            attn_scale=ATTN_SCALE, device=dev, shard=shard, ctx_dtype=torch.bfloat16,
                            result=args.result)
    n_sets = 4  # rotating query sets so consecutive steps differ
    dev_q = [make_decode_queries(B, HEADS, seed=100 + i, device=dev) for i in range(n_sets)]
    host_q = [make_decode_queries(B, HEADS, seed=100 + i, pinned=True) for i in range(n_sets)]

    def run_eager(i):
        q_idx, w, q_lat = dev_q[i % n_sets]
        return step.run(q_idx, w, q_lat, state.k_cache, state.context_lens, state.block_table, state.kv,
                        state.kv_row_base, state.context_lens_local)

    if world > 1:
        dist.barrier()                    # ranks build their state at different speeds; the kernels' waits
        torch.cuda.synchronize()          # for peers are bounded to about a second
    for i in range(2):
        res = run_eager(i)                # lazy initialisation (NCCL communicators, function attributes)
    ctx_dtype = res[1].dtype              # bf16, the dtype the reference op returns
    torch.cuda.synchronize()
    graphed = None
    if not args.no_graph:
        graphed = GraphedDecodeStep(step, state.k_cache, state.context_lens, state.block_table, state.kv,
                                    state.kv_row_base, state.context_lens_local).capture()

    from transarch_b200.decode import PipelinedDecode, input_layout, pack_inputs, unpack_inputs
    dev_pack = [pack_inputs(*dq) for dq in dev_q]       # the query sets, resident in HBM in the packed layout

    def run_device(i):
        # inputs already resident in HBM: one device-to-device copy into the graph's static buffer
        if graphed is None:
            return run_eager(i)
        return graphed.replay_packed(dev_pack[i % n_sets])

    # End to end with HOST buffers, as a serving loop would run it: three streams and four slots, so the
    # pinned-host -> device copy of step i+1 and the device -> host copy of step i-1 overlap the
    # kernels of step i.  Every step's inputs cross PCIe and every step's result reaches the host.
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    slots = 4
    # a step's three inputs travel as one packed byte buffer: one pinned arena per query set on the host, one
    # staging buffer per slot on the device (the views below are what an eager step reads)
    lay = input_layout(B, HEADS)
    host_pack = [pack_inputs(*hq, out=torch.empty(lay["bytes"], dtype=torch.uint8).pin_memory()) for hq in host_q]
    in_pack = [torch.empty(lay["bytes"], dtype=torch.uint8, device=dev) for _ in range(slots)]
    in_dev = [list(unpack_inputs(b, B, HEADS)) for b in in_pack]
    out_dev = [(torch.empty(B, TOPK, dtype=torch.int32, device=dev),
                torch.empty(B, HEADS, 512, dtype=ctx_dtype, device=dev)) for _ in range(slots)]
    out_host = [(torch.empty(B, TOPK, dtype=torch.int32).pin_memory(),
                 torch.empty(B, HEADS, 512, dtype=ctx_dtype).pin_memory()) for _ in range(slots)]
    ev_in = [torch.cuda.Event() for _ in range(slots)]
    ev_done = [torch.cuda.Event() for _ in range(slots)]
    ev_out = [torch.cuda.Event() for _ in range(slots)]
    ev_in_free = [torch.cuda.Event() for _ in range(slots)]
    e2e_started = [False] * slots

    # Sharded: the queries are replicated, but only 1/world of their bytes crosses each rank's host link;
    # an NVLink all-gather (posted peer stores, one kernel) replicates them inside the node.  Each rank
    # returns its 1/world of the result rows to its host.
    ag = None
    ag_packed = False
    if world > 1 and step.peer is not None:
        from transarch_b200.peer import PeerAllGather
        sizes = [t.numel() * t.element_size() for t in host_q[0]]
        offs = [sum(sizes[:j]) for j in range(len(sizes))]
        total_in = sum(sizes)
        ag = PeerAllGather(total_in, dev, n_send=slots)
        host_cat = []
        for hq in host_q:                                           # one pinned byte buffer per query set
            cat = torch.empty(ag.chunk * world, dtype=torch.uint8).pin_memory()
            for t, o in zip(hq, offs):
                cat[o:o + t.numel() * t.element_size()] = t.contiguous().view(torch.uint8).reshape(-1)
            host_cat.append(cat)
        recv_views = [ag.recv[o:o + n].view(t.dtype).view(t.shape) for t, o, n in zip(host_q[0], offs, sizes)]
        ag_packed = tuple(offs) == lay["offsets"] and total_in == lay["bytes"]
        rows_lo, rows_hi = rank * B // world, (rank + 1) * B // world

    # everything an iteration touches is bound once: views of the per-slot buffers (the sharded form moves only this
    # rank's rows), so that the loop itself is a handful of copy, event and launch calls
    if ag is not None:
        send_src = [hc[rank * ag.chunk:(rank + 1) * ag.chunk] for hc in host_cat]
        recv_packed = ag.recv[:lay["bytes"]] if ag_packed else None
        od = [(o[0][rows_lo:rows_hi], o[1][rows_lo:rows_hi]) for o in out_dev]
        oh = [(o[0][rows_lo:rows_hi], o[1][rows_lo:rows_hi]) for o in out_host]
    else:
        od, oh = out_dev, out_host
    res_rows = None
    if graphed is not None and graphed.out is not None:
        r_idx, r_ctx = graphed.out[0], graphed.out[1]
        res_rows = (r_idx[rows_lo:rows_hi], r_ctx[rows_lo:rows_hi]) if ag is not None else (r_idx, r_ctx)

    # Single GPU: three captured steps with buffers of their own (PipelinedDecode), so that the copies from and to
    # the host use the graphs' own buffers and no device-side staging copy is left in the loop.  (Two would stall:
    # a slot's input copy can only start once its previous result has reached the host, 160 us after its kernels,
    # and takes 190 us itself, more than the one step in between.)
    pipe = None
    if world == 1 and graphed is not None:
        captured = [graphed]
        for _ in range(2):
            step_n = SparseDecodeStep(B, shard_len, page_size=PAGE, topk=TOPK, n_heads=HEADS, index_scale=INDEX_SCALE,
                                      attn_scale=ATTN_SCALE, device=dev, shard=shard, ctx_dtype=torch.bfloat16,
                                      result=args.result)
            step_n.run(*dev_q[0], state.k_cache, state.context_lens, state.block_table, state.kv, state.kv_row_base,
                       state.context_lens_local)
            torch.cuda.synchronize()
            captured.append(GraphedDecodeStep(step_n, state.k_cache, state.context_lens, state.block_table, state.kv,
                                              state.kv_row_base, state.context_lens_local).capture())
        pipe = PipelinedDecode(captured)
        out_host = pipe.host_out              # what the byte counts below and the parity check read

    def run_e2e(i):
        if pipe is not None:
            pipe.submit(host_pack[i % n_sets])
            return
        sl = i % slots
        main = torch.cuda.current_stream()
        if e2e_started[sl]:
            ev_out[sl].synchronize()                     # result of step i-2 is on the host
            s_in.wait_event(ev_in_free[sl])
        with torch.cuda.stream(s_in):
            if ag is not None:
                ag.send[sl].copy_(send_src[i % n_sets], non_blocking=True)
            else:
                in_pack[sl].copy_(host_pack[i % n_sets], non_blocking=True)
            ev_in[sl].record(s_in)
        main.wait_event(ev_in[sl])
        if ag is not None:
            ag.run(sl)
            ins = recv_views
        else:
            ins = in_dev[sl]
        if graphed is None:
            idx, c, _ = step.run(ins[0], ins[1], ins[2], state.k_cache, state.context_lens,
                                 state.block_table, state.kv, state.kv_row_base, state.context_lens_local)
            src = (idx[rows_lo:rows_hi], c[rows_lo:rows_hi]) if ag is not None else (idx, c)
        else:
            if ag is None:
                graphed.replay_packed(in_pack[sl])
            elif ag_packed:
                graphed.replay_packed(recv_packed)       # the gathered bytes already have the layout
            else:
                graphed.replay(*ins)
            src = res_rows
        ev_in_free[sl].record(main)
        od[sl][0].copy_(src[0], non_blocking=True)
        od[sl][1].copy_(src[1], non_blocking=True)
        ev_done[sl].record(main)
        s_out.wait_event(ev_done[sl])
        with torch.cuda.stream(s_out):
            oh[sl][0].copy_(od[sl][0], non_blocking=True)
            oh[sl][1].copy_(od[sl][1], non_blocking=True)
            ev_out[sl].record(s_out)
        e2e_started[sl] = True

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, stage_events=None):
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            fn(i)
        e1.record()
        sync_all()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    for i in range(max(args.warmup, 3)):
        run_device(i)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    total_ms = timed(run_device, args.steps)
    long_steps = max(args.steps, 500)            # a second, longer timed region (also feeds the clock sampler)
    long_ms = timed(run_device, long_steps)
    clocks = sampler.stop() if rank == 0 else None
    ms_per_step = total_ms / args.steps
    value = B * args.steps / (total_ms * 1e-3)

    # per-stage device times inside a second timed region (events around each stage of the step, eager
    # launches: these include the host's launch gaps; the graph-replayed figures follow)
    stage_ms = {}

    def add(name, a, b_):
        stage_ms[name] = stage_ms.get(name, 0.0) + a.elapsed_time(b_)

    sync_all()
    for i in range(args.steps):
        q_idx, w, q_lat = dev_q[i % n_sets]
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(5)]
        ev[0].record()
        idx = step.select(q_idx, w, state.k_cache, state.context_lens_local, state.block_table)
        ev[1].record()
        if world > 1:
            idx = step.merge_candidates()
        ev[2].record()
        step.attend(q_lat, state.kv, state.kv_row_base, idx, state.context_lens, q_pos_bias=-1)
        ev[3].record()
        if world > 1:
            step.combine()
        ev[4].record()
        torch.cuda.synchronize()
        for nm, a, b_ in (("select", ev[0], ev[1]), ("exchange+merge", ev[1], ev[2]), ("attention", ev[2], ev[3]),
                          ("combine", ev[3], ev[4])):
            add(nm, a, b_)
    if world == 1:
        # the unfused pair, for comparison: indexer writing logits, then the split top-k reading them
        K = step.K
        scratch = step.topk_scratch if step.topk_scratch is not None else K.topk_scratch(B, dev)
        for i in range(args.steps):
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
            ev[0].record()
            K.indexer_paged_fp8_logits(step.q_fp8, step.weights, state.k_cache, PAGE, state.context_lens_local,
                                       state.block_table, max_cols=step.max_cols, out=step.logits)
            ev[1].record()
            K.topk_select_split(step.logits, TOPK, scratch, col_end=state.context_lens_local, sorted=False,
                                out=step.cand[:, :TOPK], out_values=step.cand[:, TOPK:].view(torch.float32))
            ev[2].record()
            torch.cuda.synchronize()
            add("unfused_indexer", ev[0], ev[1]); add("unfused_topk_split", ev[1], ev[2])
    for k_ in stage_ms:
        stage_ms[k_] /= args.steps

    # Selection alone (q quantisation + indexer + top-k), replayed from its own CUDA graph: the
    # "indexer + top-k per step" figure without the host's launch gaps of the eager stage split above.
    select_us = None
    partial_us = {}
    attention_kernels_us = None

    def graph_time(fn):
        """us per replay of fn captured into its own CUDA graph (max over ranks)."""
        s_cap = torch.cuda.Stream(device=dev)
        s_cap.wait_stream(torch.cuda.current_stream())
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.stream(s_cap):
            with torch.cuda.graph(gr, stream=s_cap):
                fn()
        torch.cuda.current_stream().wait_stream(s_cap)
        for _ in range(3):
            gr.replay()
        sync_all()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record()
        for _ in range(args.steps):
            gr.replay()
        g1.record()
        torch.cuda.synchronize()
        ms = g0.elapsed_time(g1) / args.steps
        if world > 1:
            ts = torch.tensor([ms], device=dev)
            dist.all_reduce(ts, op=dist.ReduceOp.MAX)
            ms = float(ts.item())
        gr.reset()
        return 1e3 * ms

    if graphed is not None:
        sel_q, sel_w, sel_lat = dev_q[0]

        def do_select():
            return step.select(sel_q, sel_w, state.k_cache, state.context_lens_local, state.block_table)

        select_us = graph_time(do_select)
        if world == 1:
            # the two attention kernels by themselves, each from a graph of its own: the head-split kernel the step
            # uses (M = 64) and the cluster-of-two kernel that reaches M = 128 by exchanging partial scores
            att_idx = do_select().clone()
            att_ctx = torch.empty(B, sel_lat.shape[1], 512, dtype=torch.bfloat16, device=dev)
            att_lse = torch.empty(B, sel_lat.shape[1], dtype=torch.float32, device=dev)

            def attend_with(pair):
                return lambda: step.K.sparse_mla_decode(sel_lat, state.kv, att_idx, step.attn_scale,
                                                        kv_row_base=state.kv_row_base, q_pos=state.context_lens,
                                                        q_pos_bias=-1, ctx=att_ctx, lse=att_lse, pair=pair)

            attention_kernels_us = {"heads_split_m64": round(graph_time(attend_with(False)), 2),
                                    "cluster_pair_m128": round(graph_time(attend_with(True)), 2)}
            del att_idx, att_ctx, att_lse
        if world > 1:
            # prefixes of the sharded step, each from its own graph: the differences are the exchange stages
            # Every prefix ends with a node barrier (its own kernel) so that no rank starts the next replay
            # while a peer still reads what the replay overwrites; the barrier alone is timed and subtracted.
            def fence():
                if step.peer is not None:
                    step.peer.barrier(slot=3)

            def only_fence():
                fence()

            def select_fenced():
                do_select()
                fence()

            def upto_merge():
                do_select()
                step.merge_candidates()
                fence()

            def upto_attend():
                do_select()
                idx_ = step.merge_candidates()
                step.attend(sel_lat, state.kv, state.kv_row_base, idx_, state.context_lens, q_pos_bias=-1,
                            signal=False)
                fence()

            t_fence = graph_time(only_fence) if step.peer is not None else 0.0
            t_sel = graph_time(select_fenced) - t_fence
            t_merge = graph_time(upto_merge) - t_fence
            t_att = graph_time(upto_attend) - t_fence
            partial_us = {"select": round(t_sel, 2), "exchange+merge": round(t_merge - t_sel, 2),
                          "attention": round(t_att - t_merge, 2),
                          "combine": round(1e3 * ms_per_step - t_att, 2), "node_barrier_alone": round(t_fence, 2)}

    # The dominant kernel by itself: back-to-back launches on the current stream between two events
    # (the per-stage times above include the host-side gaps of eager launches; these do not).
    reps = max(20, min(200, args.steps))
    sync_all()
    k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    k0.record()
    for _ in range(reps):
        step.K.indexer_paged_fp8_logits(step.q_fp8, step.weights, state.k_cache, PAGE, state.context_lens_local,
                                        state.block_table, max_cols=step.max_cols, out=step.logits)
    k1.record()
    torch.cuda.synchronize()
    indexer_ms = k0.elapsed_time(k1) / reps
    if world > 1:
        tt = torch.tensor([indexer_ms], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        indexer_ms = float(tt.item())
    stage_ms["indexer_back_to_back"] = indexer_ms

    # what the host link gives by itself: the step's input copy alone, back to back (explains e2e when
    # the copies, not the kernels, bound the pipelined loop)
    sync_all()
    c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    c0.record()
    for _ in range(20):
        in_pack[0].copy_(host_pack[0], non_blocking=True)
    c1.record()
    torch.cuda.synchronize()
    h2d_only_ms = c0.elapsed_time(c1) / 20

    for i in range(3):
        run_e2e(i)
    e2e_ms = timed(run_e2e, args.steps)
    e2e_value = B * args.steps / (e2e_ms * 1e-3)
    status = _lib.read_status(dev)

    # parity of the benchmarked step itself, outside every timed region (single GPU: the whole key range is here)
    parity = None
    if rank == 0 and world == 1 and not args.skip_parity:
        res = run_eager(0)
        torch.cuda.synchronize()
        try:
            parity = parity_check(step, state, dev_q[0], res, ctx, [0, B // 3, (2 * B) // 3, B - 1])
        except AssertionError as e:
            parity = {"ok": False, "error": str(e)[:300]}

    if rank == 0:
        peaks, peak_kind = measured_peaks()
        idx_bytes = B * shard_len * (128 + 4)  # fp8 key + fp32 scale per key, read once
        achieved = idx_bytes / (indexer_ms * 1e-3) / 1e9
        h2d = sum(t.numel() * t.element_size() for t in host_q[0])
        d2h = sum(t.numel() * t.element_size() for t in out_host[0])
        e2e_note = "every step: inputs from pinned host memory, indices and bf16 context back to the host"
        if ag is not None:
            e2e_note = (f"per rank and step: {ag.chunk} input bytes over the host link (1/{world} of the replicated "
                        f"queries, replicated inside the node by an NVLink all-gather kernel) and 1/{world} of the "
                        "result rows back; the byte counts below are the node totals")
        # our kernels per step: q quantisation, indexer + select (fused: 2 launches; else indexer and a top-k of
        # 3 kernels in the split form), attention; sharded:
        # + merge top-k, compaction and either barrier + peer combine or the bf16 share kernel (NCCL's
        # own kernels are not counted)
        launches = 1 + (2 if step.fused_scratch is not None else 1 + (3 if step.topk_scratch is not None else 1)) + 1
        if world > 1:
            launches += 2 + (2 if step.peer is not None else 1)
        line = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "ms_per_step_long": long_ms / long_steps,
            "steps_long": long_steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "fp8(e4m3) index scores / bf16 attention, fp32 accumulate",
            "data": "synthetic",
            "config": {"workload": WORKLOAD if (B, ctx) == (BATCH, CONTEXT) else f"batch {B}, context {ctx} (non-default)",
                       "parallelism": f"key-sharded x{world}",
                       "result": "n/a" if world == 1 else args.result,
                       "exchange": "none" if world == 1 else ("peer memory (NVLink loads/stores in our kernels)"
                                                              if step.peer is not None else "NCCL"),
                       "launch": "eager" if graphed is None else "cuda-graph replay",
                       "l2": "inputs larger than L2 (index-key cache %.2f GB per GPU, 4 rotating query sets)"
                             % (idx_bytes / 1e9)},
            "indexer_topk_us_per_step": select_us if select_us is not None else 1e3 * stage_ms["select"],
            # bytes the selection must move: keys + scales read, logits written once and read once
            "indexer_topk_hbm_frac": (None if select_us is None else
                                      (B * shard_len * (132 + 8)) / (select_us * 1e-6) / 1e9 / peaks["hbm_gbs"]),
            "stage_us": {k_: round(1e3 * v, 2) for k_, v in stage_ms.items()},
            "graph_stage_us": partial_us,
            "attention_kernels_us": attention_kernels_us,
            "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms / args.steps, "note": e2e_note, "h2d_copy_alone_ms": h2d_only_ms,
                    "h2d_copy_alone_gbs": h2d / (h2d_only_ms * 1e-3) / 1e9},
            "gpu_launches": launches * args.steps,
            "roofline": {"kernel": "indexer_paged_kernel<fp8>", "bound": "hbm", "achieved": achieved,
                         "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                         "peak_source": peak_kind, "traffic": None,
                         "timing": f"{reps} back-to-back launches of the kernel between two CUDA events, inputs larger than L2"},
            "clocks": clocks, "status_word": status,
        }
        line["roofline"]["traffic"] = DRAM_BYTES_PER_KEY * B * shard_len
        line["parity"] = parity
        threads = os.cpu_count() or 1
        if world == 1 and not args.skip_cpu_baseline:
            _, dt4, _ = cpu_tokens_per_s(4, ctx, threads)            # calibrate: about 15 s of CPU work
            n_req = max(4, min(2048, int(15.0 / max(dt4 / 4, 1e-4))))
            v, dt, kind = cpu_tokens_per_s(n_req, ctx, threads)
            line["cpu_baseline"] = {"value": v, "unit": "tokens/s", "cores": threads, "kind": kind,
                                    "sample": f"{n_req} requests of the {B}-request batch shape at context {ctx}, "
                                              f"all stages (quantise, score, top-k, attention), {dt:.1f} s"}
        if world == 1 and not args.skip_configs:
            # the rate at which the indexer's own bytes can be read at all: the pages of the cache in
            # block-table order through bare bulk copies (two pages per ring slot, as the kernel loads them)
            pages = state.block_table[:, :(shard_len + state.page_size - 1) // state.page_size].reshape(-1).long()
            offs = (pages * (state.page_size * 132)).contiguous()
            gbs = step.K.hbm_read_gbs(state.k_cache, offs, state.page_size * 132, chunks_per_stage=2)
            line["roofline"]["read_probe"] = {
                "gbs": round(gbs, 1), "frac_of_probe": round(line["roofline"]["achieved"] / gbs, 4),
                "how": "the same pages in block-table order pulled into a five-slot shared-memory ring by bare "
                       "bulk copies, two CTAs per SM, nothing computed and nothing written"}
            # tensor-pipe denominators from the library's own probe kernel, then the other configurations
            # (the decode state is released first: the configurations build their own)
            fp8_peak = step.K.mma_peak_tflops(True, device=dev)
            bf16_peak = step.K.mma_peak_tflops(False, device=dev)
            line["tensor_peaks"] = {"fp8_tflops_probe": round(fp8_peak, 1), "bf16_tflops_probe": round(bf16_peak, 1),
                                    "how": "back-to-back M=128 N=256 tcgen05 MMAs on shared-memory operands, one CTA "
                                           "per SM, best of 5 launches of about 2 ms"}
            # which bf16 instruction shapes run at the full rate of the pipe (SM clocks per instruction, counted
            # inside the kernel): the table the attention kernel's tile choice rests on
            shapes = {}
            for m_, n_, ts_ in ((128, 256, False), (128, 64, False), (128, 64, True), (64, 256, False), (64, 64, True)):
                clk = step.K.mma_shape_clocks(m_, n_, ts_, device=dev)
                shapes[f"M{m_} N{n_} K16 A-{'tmem' if ts_ else 'smem'}"] = {
                    "clocks": round(clk, 1), "flops_per_sm_clock": round(2.0 * m_ * n_ * 16 / clk)}
            line["tensor_peaks"]["bf16_shapes"] = shapes
            graphed = None
            del state, step, dev_q, in_dev, out_dev
            torch.cuda.empty_cache()
            try:
                line["configs"] = bench_configs(dev, peaks, threads, fp8_peak)
            except Exception as e:  # noqa: BLE001 - the headline line must still be printed
                line["configs"] = {"error": f"{type(e).__name__}: {e}"[:300]}
        print(json.dumps(line), flush=True)
    if world > 1:
        # A captured graph that holds NCCL kernels keeps the communicator busy: tearing the process
        # group down while it exists never returns.  Release the graph first; then leave without
        # running the communicator's destructor at all (every rank has printed and synchronised).
        if graphed is not None:
            graphed.graph.reset()
            graphed = None
        torch.cuda.synchronize()
        dist.barrier()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


if __name__ == "__main__":
    main()
