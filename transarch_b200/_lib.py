"""ctypes binding of libb200dsa.so (the C ABI declared in include/b200dsa.h).

There is no fallback: if the library is missing or a call is rejected, an exception is
raised.  Tensors are passed as raw device pointers on torch's current CUDA stream.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import torch

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libb200dsa.so")

_vp, _i32, _i64, _f32 = C.c_void_p, C.c_int32, C.c_int64, C.c_float

# name -> argtypes, in the order of include/b200dsa.h
SIGNATURES = {
    "b200dsa_abi_version": [],
    "b200dsa_last_error": [],
    "b200dsa_mma_peak_probe": [_i32, _i32, _i32, _vp, _vp],
    "b200dsa_mma_shape_probe": [_i32, _i32, _i32, _i32, _i32, _vp, _vp, _vp],
    "b200dsa_hbm_read_probe": [_vp, _vp, _i32, _i32, _i32, _i32, _vp, _vp],
    "b200dsa_topk_select": [_vp, _i64, _i32, _i32, _vp, _vp, _i32, _i32, _i32, _vp, _i64, _vp, _i64, _i32, _vp,
                            _i32, _i64, _vp, _vp, _vp, _i64, _vp],
    "b200dsa_topk_select_split": [_vp, _i64, _i32, _i32, _vp, _vp, _i32, _i32, _i32, _vp, _i32, _vp, _vp,
                                  _vp, _vp, _i64, _vp],
    "b200dsa_topk_select_split_static": [_vp, _i64, _i32, _i32, _vp, _vp, _i32, _i32, _i32, _vp, _i32,
                                         _vp, _vp, _i64, _vp],
    "b200dsa_indexer_paged_fp8_logits": [_vp, _vp, _vp, _i32, _i32, _vp, _vp, _i64, _vp, _i32, _i32, _i32, _f32,
                                         _vp, _i64, _vp, _vp, _vp, _vp],
    "b200dsa_indexer_paged_blocklist_fp8_logits": [_vp, _vp, _vp, _i32, _i32, _vp, _vp, _i64, _vp, _i32, _i32, _vp, _i64,
                                                   _vp, _i32, _f32, _vp, _i64, _vp, _vp],
    "b200dsa_indexer_paged_fp8_topk": [_vp, _vp, _vp, _i32, _i32, _vp, _vp, _i64, _vp, _i32, _i32, _i32, _f32,
                                       _vp, _i64, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _i64, _vp, _vp],
    "b200dsa_indexer_blocklist_bf16_logits": [_vp, _vp, _vp, _i32, _vp, _i64, _vp, _vp, _vp, _i32, _i32, _f32,
                                              _vp, _i64, _vp, _vp, _vp, _vp],
    "b200dsa_indexer_flat_bf16_logits": [_vp, _vp, _vp, _i32, _vp, _vp, _vp, _i32, _i32, _f32, _vp, _i64, _vp, _vp],
    "b200dsa_indexer_flat_bf16_logits_routed": [_vp, _vp, _vp, _i32, _vp, _vp, _vp, _i32, _i32, _f32, _vp, _i64, _vp, _vp],
    "b200dsa_indexer_gather_bf16_logits": [_vp, _vp, _vp, _i32, _vp, _i64, _vp, _vp, _vp, _i32, _i32, _f32, _vp, _i64,
                                           _vp, _vp],
    "b200dsa_causal_row_intervals": [_vp, _i32, _vp, _i32, _vp, _vp, _vp, _vp, _vp],
    "b200dsa_compact_owned": [_vp, _i64, _i32, _i32, _i32, _i32, _vp, _i64, _vp, _vp],
    "b200dsa_sparse_mla_decode": [_vp, _vp, _i64, _vp, _vp, _i64, _i32, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _f32,
                                  _vp, _i32, _vp, _vp, _vp],
    "b200dsa_sparse_mla_decode_pair": [_vp, _vp, _i64, _vp, _vp, _i64, _i32, _vp, _vp, _i32, _i32, _i32, _i32, _i32,
                                       _f32, _vp, _i32, _vp, _vp, _vp],
    "b200dsa_wuv_up_project": [_vp, _vp, _i32, _i32, _i32, _vp, _i32, _vp, _vp],
    "b200dsa_lse_combine": [_vp, _vp, _i32, _i64, _vp, _vp, _vp],
    "b200dsa_peer_lse_combine": [_vp, _i32, _i32, _i64, _i64, _i64, _i64, _i64, _i64, _vp, _i32, _i32, _i32, _vp, _vp],
    "b200dsa_indexer_paged_fp8_topk_push": [_vp, _vp, _vp, _i32, _i32, _vp, _vp, _i64, _vp, _i32, _i32, _i32, _f32,
                                            _vp, _i64, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _i64, _vp, _i64, _vp, _vp],
    "b200dsa_topk_merge_owned": [_vp, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _i64, _vp, _i64, _vp, _vp, _vp, _vp],
    "b200dsa_sparse_mla_decode_signal": [_vp, _vp, _i64, _vp, _vp, _i64, _i32, _vp, _vp, _i32, _i32, _i32, _i32, _i32,
                                         _f32, _vp, _i32, _vp, _vp, _vp, _vp, _vp],
    "b200dsa_peer_barrier": [_vp, _i32, _i32, _i64, _i32, _vp, _vp, _vp],
    "b200dsa_peer_gather": [_vp, _i32, _i32, _i64, _i64, _vp, _i64, _i32, _vp, _vp, _vp],
    "b200dsa_peer_push": [_vp, _i32, _i32, _i64, _i64, _i64, _i64, _i32, _vp, _vp, _vp],
    "b200dsa_peer_set_wait_limit": [_i64],
    "b200dsa_peer_alloc": [_i64, _vp, _vp],
    "b200dsa_peer_open": [_vp, _vp],
    "b200dsa_peer_close": [_vp],
    "b200dsa_peer_free": [_vp],
    "b200dsa_lse_prescale": [_vp, _vp, _vp, _i64, _vp, _vp],
    "b200dsa_lse_finalize": [_vp, _vp, _i64, _vp, _vp, _vp],
    "b200dsa_lse_prescale_norm": [_vp, _vp, _i32, _i32, _i64, _vp, _vp, _vp],
    "b200dsa_quant_q_fold_weights": [_vp, _vp, _i64, _f32, _i32, _vp, _vp, _vp],
    "b200dsa_indexer_k_norm_rope": [_vp, _i32, _i64, _vp, _vp, _f32, _vp, _vp, _i32, _vp, _vp, _vp, _i64, _i32, _i32,
                                    _vp, _vp],
    "b200dsa_indexer_q_rope": [_vp, _i32, _i64, _i32, _vp, _vp, _i32, _vp, _vp, _f32, _i32, _vp, _vp, _vp],
    "b200dsa_block_mean_pool_bf16": [_vp, _i32, _i32, _vp, _vp, _vp],
    "b200dsa_paged_mean_pool_fp8": [_vp, _i32, _i32, _vp, _vp, _i64, _i32, _i32, _i32, _vp, _vp, _vp],
    "b200dsa_sparse_attn_bwd_pointwise": [_vp, _vp, _i32, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _f32, _vp, _vp, _vp],
    "b200dsa_scatter_add_latent_rows": [_vp, _i64, _vp, _vp, _i32, _vp, _vp, _i32, _i32, _vp, _vp],
    "b200dsa_paged_mean_pool_fp8_update": [_vp, _i32, _i32, _vp, _vp, _vp, _i64, _i32, _i32, _i32, _i32, _vp, _vp,
                                           _vp, _vp],
    "b200dsa_router_qnorm_topk": [_vp, _vp, _i32, _i32, _vp, _vp, _vp],
    "b200dsa_router_block_score_topk": [_vp, _vp, _vp, _i64, _vp, _vp, _vp, _i32, _i32, _vp, _vp, _vp, _vp],
    "b200dsa_router_linear_topk_softmax": [_vp, _vp, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _vp],
    "b200dsa_indexer_k_quant_and_cache": [_vp, _vp, _i64, _vp, _i64, _i32, _i32, _vp, _vp],
}



class PeerLink(C.Structure):
    """b200dsa_peer_link of include/b200dsa.h."""
    _fields_ = [("bufs", C.c_void_p), ("rank", C.c_int32), ("world", C.c_int32), ("off_flags", C.c_int64),
                ("slot", C.c_int32), ("state", C.c_void_p)]


_lib: Optional[C.CDLL] = None


class B200DSAError(RuntimeError):
    pass


def load() -> C.CDLL:
    """Load the library (once).  Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise B200DSAError(
            f"{LIB_PATH} is missing: build it with `python -m transarch_b200.build` "
            "(there is no CPU or PyTorch fallback for these kernels)")
    lib = C.CDLL(LIB_PATH)
    for name, argtypes in SIGNATURES.items():
        fn = getattr(lib, name)           # AttributeError if the symbol is not exported
        fn.argtypes = argtypes
        fn.restype = C.c_char_p if name == "b200dsa_last_error" else C.c_int
    _lib = lib
    return lib


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = load().b200dsa_last_error()
        raise B200DSAError(f"{what} failed with code {rc}: {msg.decode() if msg else ''}")


def require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise B200DSAError("b200dsa kernels need CUDA tensors; there is no CPU path")


_status_words = {}


def status_word(device: torch.device) -> torch.Tensor:
    """Per-device int32 status word the kernels raise on bounded-wait timeouts / bad indices."""
    key = (device.type, device.index if device.index is not None else torch.cuda.current_device())
    if key not in _status_words:
        _status_words[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status_words[key]


def read_status(device: torch.device) -> int:
    """Synchronising read-and-clear of the status word (tests and debugging only)."""
    w = status_word(device)
    v = int(w.item())
    if v:
        w.zero_()
    return v
