"""The library's measurement kernels: they must run, give the status word back clean, and report
figures of the right order (the bench line quotes them as roofline denominators)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_tensor_probes_run():
    from transarch_b200 import _lib, kernels as K
    fp8 = K.mma_peak_tflops(True, iters=2048, reps=2)
    bf16 = K.mma_peak_tflops(False, iters=2048, reps=2)
    assert 700 < bf16 < 2700 and 1.5 < fp8 / bf16 < 2.3, (fp8, bf16)
    full = K.mma_shape_clocks(128, 256, False, iters=512)
    half = K.mma_shape_clocks(64, 256, False, iters=512)
    assert 115 < full < 150 and 115 < half < 150, (full, half)   # M = 64 takes the time of M = 128: half the rate
    with pytest.raises(_lib.B200DSAError):
        K.mma_shape_clocks(96, 64, False)
    assert _lib.read_status(torch.device("cuda")) == 0


def test_hbm_read_probe_runs():
    from transarch_b200 import _lib, kernels as K
    page = 64 * 132
    n_pages = 32768                                           # 277 MB, larger than L2
    buf = torch.zeros(n_pages * page, dtype=torch.uint8, device="cuda")
    order = torch.randperm(n_pages, device="cuda")
    gbs = K.hbm_read_gbs(buf, (order * page).contiguous(), page, chunks_per_stage=2, reps=5)
    assert 1500 < gbs < 9000, gbs
    with pytest.raises(_lib.B200DSAError):
        K.hbm_read_gbs(buf, (order * page).contiguous(), page, chunks_per_stage=3)   # 3 x 8448 bytes do not fit a ring slot
    assert _lib.read_status(torch.device("cuda")) == 0
