"""Host-side logic that needs no GPU: the packed input layout of the decode step and the backward
arithmetic of the differentiable sparse attention (its kernels replaced by the oracle's forward)."""
import torch

from oracle import dsa_oracle as O


def test_packed_input_layout_round_trip():
    from transarch_b200.decode import input_layout, pack_inputs, unpack_inputs
    B, H = 5, 16
    lay = input_layout(B, H)
    assert all(o % 256 == 0 for o in lay["offsets"]) and lay["bytes"] % 256 == 0
    assert lay["sizes"] == (B * 64 * 128 * 2, B * 64 * 4, B * H * 576 * 2)
    g = torch.Generator().manual_seed(0)
    q_idx = torch.randn(B, 64, 128, generator=g).bfloat16()
    w = torch.randn(B, 64, generator=g)
    q_lat = torch.randn(B, H, 576, generator=g).bfloat16()
    buf = pack_inputs(q_idx, w, q_lat)
    assert buf.dtype == torch.uint8 and buf.numel() == lay["bytes"]
    a, b, c = unpack_inputs(buf, B, H)
    assert torch.equal(a, q_idx) and torch.equal(b, w) and torch.equal(c, q_lat)
    # views, not copies: writing through them changes the packed buffer
    b.zero_()
    assert unpack_inputs(buf, B, H)[1].abs().sum() == 0


def test_sparse_attention_backward_arithmetic(monkeypatch):
    """The backward pass rebuilds p = exp(s - lse) from the saved log-sum-exp and runs five products per query
    chunk; with the forward kernels replaced by the oracle's fp32 forward its gradients must equal autograd
    through the oracle's own op (fp32, several chunk sizes, -1 padding, future positions, an empty row)."""
    from transarch_b200 import opendsa_ops as D
    g = torch.Generator().manual_seed(3)
    L, H, Dl, d_c, K, Dv = 23, 4, 576, 512, 11, 6
    q = torch.randn(L, H, Dl, generator=g) * 0.3
    lat = torch.randn(L, Dl, generator=g) * 0.3
    W = torch.randn(H, Dv, d_c, generator=g) / d_c ** 0.5
    idx = torch.randint(0, L, (L, K), generator=g)
    idx[torch.rand(L, K, generator=g) < 0.2] = -1
    idx[4] = -1                                     # a query without any key
    G = torch.randn(L, H, Dv, generator=g)
    scale = Dl ** -0.5

    def fake_latent(q_lat, latent, indices, *, sm_scale, q_pos=None, ctx_dtype=torch.float32):
        return O.sparse_attend_latent(q_lat.detach(), latent.detach(), indices, d_c=d_c, sm_scale=sm_scale, q_pos=q_pos)

    monkeypatch.setattr(D, "sparse_attend_latent", fake_latent)
    monkeypatch.setattr(D, "_up_project", lambda ctx, W_UV: torch.einsum("thl,hvl->thv", ctx.float(), W_UV.float()))
    a, b, c = (t.clone().requires_grad_() for t in (q, lat, W))
    (O.sparse_attend_absorbed(a, b, c, idx, d_c=d_c, sm_scale=scale) * G).sum().backward()
    for chunk in (5, 23, 512):
        x, y, z = (t.clone().requires_grad_() for t in (q, lat, W))
        out = D._SparseAttendAbsorbed.apply(x, y, z, idx, torch.arange(L), scale, chunk)
        (out * G).sum().backward()
        for got, ref in ((x.grad, a.grad), (y.grad, b.grad), (z.grad, c.grad)):
            assert torch.allclose(got, ref, rtol=1e-4, atol=1e-6), (chunk, float((got - ref).abs().max()))
