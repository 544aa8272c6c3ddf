"""The allocation-free split top-k (scratch built into the library) must return exactly what the
caller-scratch entry point returns, call after call.  Runs last, and also passes on its own in a
fresh process: the first call on the device performs the one-time address look-up."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_static(lib, s, lens, k, out, val, splits=4, sorted_=1):
    return lib.b200dsa_topk_select_split_static(
        s.data_ptr(), s.stride(0), s.shape[0], s.shape[1], None, lens.data_ptr(), k, 0, sorted_, None, splits,
        out.data_ptr(), val.data_ptr(), out.stride(0), torch.cuda.current_stream().cuda_stream)


def test_static_scratch_entry_matches_caller_scratch_entry_twice():
    from transarch_b200 import _lib, kernels as K
    lib = _lib.load()
    g = torch.Generator().manual_seed(2024)
    k = 2048
    for call, (rows, cols) in enumerate([(64, 40000), (9, 131072)]):      # two calls in a row, different shapes
        s = torch.randn(rows, cols, generator=g).cuda()
        lens = torch.randint(cols // 2, cols + 1, (rows,), generator=g, dtype=torch.int32).cuda()
        lens[0] = 50                                                      # a short row as well
        out = torch.empty(rows, k, dtype=torch.int32, device="cuda")
        val = torch.empty(rows, k, dtype=torch.float32, device="cuda")
        rc = _call_static(lib, s, lens, k, out, val)
        assert rc == 0, lib.b200dsa_last_error()
        scratch = K.topk_scratch(rows, s.device)
        ref_val = torch.empty(rows, k, dtype=torch.float32, device="cuda")
        ref = K.topk_select_split(s, k, scratch, col_end=lens, splits=4, out_values=ref_val)[0]
        torch.cuda.synchronize()
        assert torch.equal(out, ref), f"call {call}: indices differ"       # integer work: bit-exact
        assert torch.equal(val, ref_val), f"call {call}: values differ"
        # and once more on the same inputs: the shared array carries state from the call before
        out2 = torch.empty_like(out)
        assert _call_static(lib, s, lens, k, out2, val) == 0
        torch.cuda.synchronize()
        assert torch.equal(out2, ref)
    # the tensor-level wrapper goes through the same entry point
    out3 = torch.empty(rows, k, dtype=torch.int32, device="cuda")
    K.topk_select_split_static(s, k, col_end=lens, splits=4, out=out3)
    assert torch.equal(out3, ref)


def test_static_scratch_entry_rejects_more_rows_than_it_holds():
    from transarch_b200 import _lib
    lib = _lib.load()
    s = torch.zeros(65, 16, device="cuda")
    lens = torch.full((65,), 16, dtype=torch.int32, device="cuda")
    out = torch.empty(65, 4, dtype=torch.int32, device="cuda")
    val = torch.empty(65, 4, dtype=torch.float32, device="cuda")
    rc = _call_static(lib, s, lens, 4, out, val)
    assert rc == -1
    assert b"64 rows" in lib.b200dsa_last_error()
