"""The lightning indexer as a module, with the reference's constructor and forward signature:

    LightningIndexer(hidden_size, n_heads, head_dim, rope_dim, q_input_dim, dtype)
    forward(hidden_states [B,L,hidden], q_input [B,L,q_in], cos [B,L,rope_dim], sin [B,L,rope_dim])
        -> q_idx [B,L,H,d], k_idx [B,L,d], w [B,L,H]
    OpenDSA/opendsa/modeling/indexer.py:40-83

Parameter names (wq, wk, k_norm, w_proj) and shapes are the reference's, so its state dict loads
unchanged.  The three dense projections are plain GEMMs (torch / cuBLAS); everything after them runs in
two fused kernels: LayerNorm + RoPE on the key rows, RoPE on the (token, head) query rows.

`forward_quantised` is the serving form of the same producer (MiSAIndexer.forward,
MISA_preprint/misa_vllm_patch_2stage/misa_vllm_patch/misa_deepseek_v2.py:228-292, where the rope dims
come FIRST): it returns the FP8 queries with their scales folded into the head weights, and writes the
new keys, quantised, straight into the paged cache.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from . import kernels as K
from ._lib import B200DSAError


class LightningIndexer(nn.Module):
    def __init__(self, hidden_size: int, n_heads: int = 8, head_dim: int = 128, rope_dim: int = 64,
                 q_input_dim: Optional[int] = None, dtype: torch.dtype = torch.bfloat16):
        super().__init__()
        if head_dim != 128 or rope_dim not in (0, 64):
            raise B200DSAError("the fused kernels need head_dim = 128 and rope_dim = 64 (or 0)")
        self.hidden_size, self.n_heads, self.head_dim, self.rope_dim = hidden_size, n_heads, head_dim, rope_dim
        self.nope_dim = head_dim - rope_dim
        q_in = q_input_dim if q_input_dim is not None else hidden_size
        self.q_input_dim = q_in
        self.softmax_scale = head_dim ** -0.5
        self.wq = nn.Linear(q_in, n_heads * head_dim, bias=False, dtype=dtype)
        self.wk = nn.Linear(hidden_size, head_dim, bias=False, dtype=dtype)
        self.k_norm = nn.LayerNorm(head_dim, dtype=dtype)
        self.w_proj = nn.Linear(hidden_size, n_heads, bias=False, dtype=dtype)

    @torch.no_grad()
    def forward(self, hidden_states, q_input, cos, sin):
        """Returns q_idx [B,L,H,d], k_idx [B,L,d], w [B,L,H] (inference only: the kernels have no backward)."""
        B, L, _ = hidden_states.shape
        H, d = self.n_heads, self.head_dim
        q = self.wq(q_input).view(B * L, H, d).contiguous()
        k = self.wk(hidden_states).view(B * L, d).contiguous()
        rope = self.rope_dim > 0
        c = cos.reshape(B * L, -1) if rope else None
        s = sin.reshape(B * L, -1) if rope else None
        q_idx = K.indexer_q_rope(q, c, s) if rope else q
        k_idx = K.indexer_k_norm_rope(k, self.k_norm.weight, self.k_norm.bias, self.k_norm.eps, c, s)
        w = self.w_proj(hidden_states) * (self.n_heads ** -0.5)
        return q_idx.view(B, L, H, d), k_idx.view(B, L, d), w

    @torch.no_grad()
    def forward_quantised(self, hidden_states, q_input, cos, sin, cache, slot_mapping, page_size: int, *,
                          scale_fmt: Optional[str] = "ue8m0", rope_first: bool = True):
        """Token-flattened inputs [T, ...]; cos / sin [T, 64].  Returns (q_fp8 [T,H,128], weights [T,H] fp32 =
        w_proj(h) * q_scale * softmax_scale * H^-0.5) and inserts the T new keys into `cache`."""
        T = hidden_states.shape[0]
        H, d = self.n_heads, self.head_dim
        q = self.wq(q_input).view(T, H, d).contiguous()
        k = self.wk(hidden_states).view(T, d).contiguous()
        w = self.w_proj(hidden_states)
        q_fp8, weights = K.indexer_q_rope(q, cos, sin, rope_first=rope_first, want_rows=False, w=w,
                                          fold=self.softmax_scale * H ** -0.5, ue8m0=scale_fmt is not None)
        K.indexer_k_norm_rope(k, self.k_norm.weight, self.k_norm.bias, self.k_norm.eps, cos, sin,
                              rope_first=rope_first, want_rows=False, cache=cache, slot_mapping=slot_mapping,
                              page_size=page_size, scale_fmt=scale_fmt)
        return q_fp8, weights
