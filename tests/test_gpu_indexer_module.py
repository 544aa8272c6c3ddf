"""The lightning-indexer module (reference signature and parameter names) against the reference module's
own outputs, and its fused serving form against the oracle's quantisers."""
import os

import numpy as np
import pytest
import torch

from oracle import dsa_oracle as O
from tests.golden.make_golden import INDEXER_CASES, golden_inputs_indexer

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


def _ref_rope(x, cos, sin, first):
    """rotate-half RoPE on the first / last 64 dims (OpenDSA/opendsa/modeling/indexer.py:27-37, :73-79)."""
    a, b = (x[..., :64], x[..., 64:]) if first else (x[..., 64:], x[..., :64])
    rot = torch.cat((-a[..., 32:], a[..., :32]), dim=-1)
    a = a * cos + rot * sin
    return torch.cat((a, b), -1) if first else torch.cat((b, a), -1)


def test_module_matches_reference_outputs_fp32():
    from transarch_b200.indexer_module import LightningIndexer
    name, seed, B, L, hidden, H = INDEXER_CASES[0]
    h, cos, sin, state = golden_inputs_indexer(seed, B, L, hidden, H)
    gold = np.load(os.path.join(GOLD, name + ".npz"))
    mod = LightningIndexer(hidden, n_heads=H, dtype=torch.float32).cuda()
    mod.load_state_dict(state)                      # the reference's parameter names, unchanged
    torch.backends.cuda.matmul.allow_tf32 = False
    q, k, w = mod(h.cuda(), h.cuda(), cos.cuda(), sin.cuda())
    for got, want in ((q, gold["q"]), (k, gold["k"]), (w, gold["w"])):
        want = torch.from_numpy(want)
        assert got.shape == want.shape
        assert (got.cpu() - want).abs().max() < 2e-4 * want.abs().max()


def test_module_bf16_and_quantised_serving_form():
    from transarch_b200 import _lib
    from transarch_b200.indexer_module import LightningIndexer
    g = torch.Generator().manual_seed(31)
    T, hidden, H, P = 50, 64, 64, 64
    mod = LightningIndexer(hidden, n_heads=H, dtype=torch.bfloat16).cuda()
    with torch.no_grad():
        mod.k_norm.weight.copy_(1.0 + 0.1 * torch.randn(128, generator=g))
        mod.k_norm.bias.copy_(0.1 * torch.randn(128, generator=g))
    h = torch.randn(T, hidden, generator=g).bfloat16().cuda()
    ang = torch.rand(T, 32, generator=g) * 6.28
    cos = torch.cat([ang.cos(), ang.cos()], -1).cuda()
    sin = torch.cat([ang.sin(), ang.sin()], -1).cuda()
    # bf16 rows of the training-side forward (rope dims last) against fp32 math on the same projections
    q, k, w = mod(h.view(1, T, hidden), h.view(1, T, hidden), cos.view(1, T, 64), sin.view(1, T, 64))
    qp = mod.wq(h).float().view(T, H, 128)
    kp = torch.nn.functional.layer_norm(mod.wk(h).float(), (128,), mod.k_norm.weight.float(), mod.k_norm.bias.float(),
                                        mod.k_norm.eps)
    q_ref = _ref_rope(qp, cos.view(T, 1, 64), sin.view(T, 1, 64), first=False)
    k_ref = _ref_rope(kp, cos, sin, first=False)
    assert (q[0].float() - q_ref).abs().max() < 1e-2 * q_ref.abs().max()
    assert (k[0].float() - k_ref).abs().max() < 1e-2 * k_ref.abs().max()
    assert torch.allclose(w[0].float(), (mod.w_proj(h) * H ** -0.5).float())
    # serving form: rope dims first, FP8 queries with folded weights, keys quantised into the cache
    n_pages = 4
    cache = torch.zeros(n_pages, P * 132, dtype=torch.uint8, device="cuda")
    slots = torch.randperm(n_pages * P, generator=g)[:T].to(torch.int64).cuda()
    q_fp8, weights = mod.forward_quantised(h, h, cos, sin, cache, slots, P, scale_fmt="ue8m0")
    assert _lib.read_status(h.device) == 0
    q_rows = _ref_rope(qp, cos.view(T, 1, 64), sin.view(T, 1, 64), first=True).bfloat16().float().cpu()
    k_rows = _ref_rope(kp, cos, sin, first=True).bfloat16().float().cpu()
    rq, rw = O.quant_q_fold_weights(q_rows, mod.w_proj(h).float().cpu(), 128 ** -0.5, H ** -0.5, ue8m0=True)
    # a bf16 rounding of the row may differ by one ulp between the fused kernel (fp32 -> bf16 once) and this
    # reference chain; compare dequantised values instead of bytes
    deq = q_fp8.float().cpu() * (weights.cpu() / (mod.w_proj(h).float().cpu() * 128 ** -0.5 * H ** -0.5)).unsqueeze(-1)
    want = rq.float() * (rw / (mod.w_proj(h).float().cpu() * 128 ** -0.5 * H ** -0.5)).unsqueeze(-1)
    assert (deq - want).abs().max() < 0.07 * want.abs().max()            # e4m3 step at the top binade: 1/16
    kq, ks = O.quant_fp8_rows(k_rows, ue8m0=True)
    c = cache.cpu()
    vals = c[:, :P * 128].reshape(-1, 128).view(torch.float8_e4m3fn).float()
    scales = c[:, P * 128:].contiguous().view(torch.float32).reshape(-1)
    sl = slots.cpu()
    got = vals[sl] * scales[sl].unsqueeze(-1)
    assert (got - kq.float() * ks.unsqueeze(-1)).abs().max() < 0.07 * k_rows.abs().max()
    m, _ = torch.frexp(scales[sl])
    assert (m == 0.5).all()                                               # power-of-two scales
