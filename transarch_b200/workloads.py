"""Seeded synthetic state for the decode path, generated on the device.

Shapes and value laws of a DeepSeek-V3.2-style decode batch: index keys N(0,1) quantised to
e4m3 with a per-token scale and packed into pages of `page_size` tokens
(page = page_size*128 fp8 bytes then page_size fp32 scales) behind a shuffled block table;
latent KV 0.5*N(0,1) bf16 [*, 576]; index queries N(0,1) bf16; head weights N(0,1)/8;
MLA queries N(0,1) bf16.  A rank of a key-sharded run generates only its own position range
(seed + rank), so no rank ever holds the whole cache.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch


@dataclass
class DecodeState:
    k_cache: torch.Tensor        # uint8 [num_pages, page_size*132]
    block_table: torch.Tensor    # int32 [B, pages_per_request]
    context_lens: torch.Tensor   # int32 [B] global context lengths
    context_lens_local: torch.Tensor  # int32 [B] keys inside this rank's range
    kv: torch.Tensor             # bf16 [B*local_len, 576]
    kv_row_base: torch.Tensor    # int64 [B]
    page_size: int
    local_len: int


def quantize_keys_fp8(k: torch.Tensor):
    """Per-token e4m3 quantisation: scale = max(amax, 1e-4)/448."""
    amax = k.float().abs().amax(dim=-1, keepdim=True).clamp_min(1e-4)
    scale = amax / 448.0
    kq = (k.float() / scale).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)
    return kq, scale.squeeze(-1)


def make_decode_state(batch: int, context_lens, *, page_size: int = 64, seed: int = 4, rank: int = 0,
                      world_size: int = 1, shard_len: Optional[int] = None,
                      device: Optional[torch.device] = None) -> DecodeState:
    """Build this rank's paged FP8 index-key cache and latent KV for `batch` requests.

    context_lens: int or sequence of per-request global lengths.  With world_size > 1 the rank
    owns positions [rank*shard_len, (rank+1)*shard_len) of every request."""
    dev = device if device is not None else torch.device("cuda")
    gen = torch.Generator(device=dev).manual_seed(seed * 1000 + rank)
    if isinstance(context_lens, int):
        context_lens = [context_lens] * batch
    lens = torch.tensor(list(context_lens), dtype=torch.int32)
    max_len = int(lens.max())
    if world_size == 1:
        shard_len = max_len
        lo = 0
    else:
        assert shard_len is not None and shard_len % page_size == 0
        lo = rank * shard_len
    local = (lens - lo).clamp(min=0, max=shard_len).to(torch.int32)
    pages_per = (shard_len + page_size - 1) // page_size
    num_pages = batch * pages_per
    cache = torch.empty(num_pages, page_size * 132, dtype=torch.uint8, device=dev)
    table = torch.randperm(num_pages, generator=gen, device=dev).view(batch, pages_per).to(torch.int32)
    kv = torch.empty(batch * shard_len, 576, dtype=torch.bfloat16, device=dev)
    for b in range(batch):  # one request at a time keeps the fp32 temporaries small
        k = torch.randn(pages_per * page_size, 128, generator=gen, device=dev)
        kq, sc = quantize_keys_fp8(k)
        pages = table[b].long()
        cache[pages, : page_size * 128] = kq.view(torch.uint8).view(pages_per, page_size * 128)
        cache[pages, page_size * 128:] = sc.contiguous().view(torch.uint8).view(pages_per, page_size * 4)
        kv[b * shard_len:(b + 1) * shard_len] = (0.5 * torch.randn(shard_len, 576, generator=gen, device=dev)).bfloat16()
    base = torch.arange(batch, dtype=torch.int64, device=dev) * shard_len
    return DecodeState(cache, table, lens.to(dev), local.to(dev), kv, base, page_size, shard_len)


def make_decode_queries(batch: int, n_heads: int = 128, *, seed: int = 4, device=None, pinned: bool = False):
    """(q_idx bf16 [B,64,128], w fp32 [B,64], q_lat bf16 [B,H,576]); identical on every rank
    for a given seed.  pinned=True returns page-locked host tensors."""
    g = torch.Generator().manual_seed(seed)
    q_idx = torch.randn(batch, 64, 128, generator=g).bfloat16()
    w = (torch.randn(batch, 64, generator=g) / 8).float()
    q_lat = torch.randn(batch, n_heads, 576, generator=g).bfloat16()
    if pinned:
        return q_idx.pin_memory(), w.pin_memory(), q_lat.pin_memory()
    dev = device if device is not None else torch.device("cuda")
    return q_idx.to(dev), w.to(dev), q_lat.to(dev)
