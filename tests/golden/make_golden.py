"""Generate golden vectors by running the reference's own OpenDSA ops on seeded inputs.

Run once where a TransArch checkout is available:
    python tests/golden/make_golden.py /path/to/TransArch
The reference is imported read-only; only its outputs (small .npz files) are stored.
Inputs are regenerated from the seeds by `golden_inputs`, so the files hold outputs only
(plus tiny inputs where the generator is not a plain randn).
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

# (name, seed, Lq, Lk, H, d, topk, docs, mode)
SELECT_CASES = [
    ("select_single_doc", 10, 96, 96, 8, 32, 16, [96], "packed"),
    ("select_packed_docs", 11, 160, 160, 64, 128, 32, [40, 1, 70, 49], "packed"),
    ("select_topk_gt_len", 12, 48, 48, 4, 16, 64, [48], "packed"),
    ("select_cp_global_pos", 13, 24, 200, 64, 128, 48, [120, 80], "cp"),
    ("select_decode_one_query", 14, 1, 777, 64, 128, 256, [777], "decode"),
]

# (name, seed, L, H, Dl, d_c, K)
ATTEND_CASES = [
    ("attend_small", 20, 64, 4, 40, 32, 16),
    ("attend_mla_shape", 21, 24, 8, 576, 512, 24),
]


# (name, seed, B, L, hidden, n_heads)
INDEXER_CASES = [
    ("lightning_indexer_fp32", 30, 2, 16, 32, 8),
]


def golden_inputs_indexer(seed, B, L, hidden, n_heads):
    """Inputs and parameters of the indexer module, all from the seed (fp32): hidden states, rotary
    cos / sin of real positions (rotate-half convention: both halves carry the same angles), and a state
    dict with the reference's parameter names."""
    g = torch.Generator().manual_seed(seed)
    h = torch.randn(B, L, hidden, generator=g)
    pos = torch.arange(L, dtype=torch.float32).view(1, L, 1) + torch.tensor([0.0, 100.0]).view(B, 1, 1)
    inv = 10000.0 ** (-torch.arange(0, 32, dtype=torch.float32) / 32.0)
    ang = torch.cat([pos * inv, pos * inv], dim=-1)
    cos, sin = ang.cos(), ang.sin()
    state = {
        "wq.weight": torch.randn(n_heads * 128, hidden, generator=g) / hidden ** 0.5,
        "wk.weight": torch.randn(128, hidden, generator=g) / hidden ** 0.5,
        "k_norm.weight": 1.0 + 0.1 * torch.randn(128, generator=g),
        "k_norm.bias": 0.1 * torch.randn(128, generator=g),
        "w_proj.weight": torch.randn(n_heads, hidden, generator=g) / hidden ** 0.5,
    }
    return h, cos, sin, state


def golden_inputs_select(seed, Lq, Lk, H, d, docs, mode):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(Lq, H, d, generator=g)
    k = torch.randn(Lk, d, generator=g)
    w = torch.randn(Lq, H, generator=g) / 8
    cu = torch.tensor([0] + list(np.cumsum(docs)), dtype=torch.int64)
    if mode == "packed":
        gpos = None
    elif mode == "cp":
        gpos = torch.sort(torch.randperm(Lk, generator=g)[:Lq]).values
    else:  # decode: one query at the last position
        gpos = torch.tensor([Lk - 1])
    return q, k, w, cu, gpos


def golden_inputs_attend(seed, L, H, Dl, d_c, K):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(L, H, Dl, generator=g)
    lat = 0.5 * torch.randn(L, Dl, generator=g)
    W_UV = torch.randn(H, 8, d_c, generator=g) / d_c ** 0.5
    # indices: random causal picks, some -1, some future (must be masked), one empty row
    idx = torch.randint(0, L, (L, K), generator=g, dtype=torch.int64)
    drop = torch.rand(L, K, generator=g) < 0.2
    idx[drop] = -1
    idx[3] = -1
    return q, lat, W_UV, idx.to(torch.int32)


def main(ref_root: str):
    sys.path.insert(0, os.path.join(ref_root, "OpenDSA"))
    from opendsa.ops import indexer_select_topk, sparse_attend_absorbed_chunked, prepare_ks_ke
    from opendsa.ops.flashkl_warmup import prepare_ks_ke_cp

    torch.manual_seed(0)
    for name, seed, Lq, Lk, H, d, topk, docs, mode in SELECT_CASES:
        q, k, w, cu, gpos = golden_inputs_select(seed, Lq, Lk, H, d, docs, mode)
        idx = indexer_select_topk(q, k, w, cu, topk, q_global_pos=gpos)
        if gpos is None:
            ks, ke = prepare_ks_ke(cu)
        else:
            ks, ke = prepare_ks_ke_cp(cu, gpos)
        np.savez_compressed(os.path.join(HERE, name + ".npz"),
                            idx=idx.numpy(), ks=ks.numpy(), ke=ke.numpy())
        print(name, tuple(idx.shape))

    for name, seed, L, H, Dl, d_c, K in ATTEND_CASES:
        q, lat, W_UV, idx = golden_inputs_attend(seed, L, H, Dl, d_c, K)
        out = sparse_attend_absorbed_chunked(q, lat, W_UV, idx, d_c=d_c, sm_scale=Dl ** -0.5,
                                             checkpoint=False, q_chunk=16)
        # identity up-projection exposes the latent-space context the kernels emit
        eye = torch.eye(d_c).unsqueeze(0).expand(H, d_c, d_c).contiguous()
        ctx = sparse_attend_absorbed_chunked(q, lat, eye, idx, d_c=d_c, sm_scale=Dl ** -0.5,
                                             checkpoint=False, q_chunk=16)
        np.savez_compressed(os.path.join(HERE, name + ".npz"),
                            out=out.numpy().astype(np.float32), ctx=ctx.numpy().astype(np.float32))
        print(name, tuple(out.shape))


def main_indexer(ref_root: str):
    sys.path.insert(0, os.path.join(ref_root, "OpenDSA"))
    from opendsa.modeling.indexer import LightningIndexer
    for name, seed, B, L, hidden, n_heads in INDEXER_CASES:
        h, cos, sin, state = golden_inputs_indexer(seed, B, L, hidden, n_heads)
        mod = LightningIndexer(hidden, n_heads=n_heads, head_dim=128, rope_dim=64, dtype=torch.float32)
        mod.load_state_dict(state)
        with torch.no_grad():
            q, k, w = mod(h, h, cos, sin)
        np.savez_compressed(os.path.join(HERE, name + ".npz"), q=q.numpy(), k=k.numpy(), w=w.numpy())
        print(name, tuple(q.shape), tuple(k.shape), tuple(w.shape))


if __name__ == "__main__":
    if len(sys.argv) > 2 and sys.argv[2] == "indexer":
        main_indexer(sys.argv[1])
        sys.exit(0)
    main(sys.argv[1] if len(sys.argv) > 1 else os.environ.get("TRANSARCH_ROOT", "."))
    main_indexer(sys.argv[1] if len(sys.argv) > 1 else os.environ.get("TRANSARCH_ROOT", "."))
