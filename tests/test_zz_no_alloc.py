"""The allocation-free GEMM entry point (collected last on purpose).

Some callers cannot allocate device memory when they need a GEMM (their own arena owns the
device, or they cannot risk the synchronisation an allocation may cause), so
strix_cuda_prefill_q8_gemm_noalloc takes all its scratch from a fixed array inside the
library. It must give what the regular device entry point gives, also on a second call that
finds the previous call's leftovers in the array, and it must refuse shapes that do not fit."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
REL_L2_TOL = 1e-3


def rel_l2(got, want):
    return float(np.linalg.norm(got.astype(np.float64) - want) / max(np.linalg.norm(want), 1e-30))


def test_noalloc_gemm_matches_regular_entry_point_twice(accel, synth, pkg):
    import torch
    dev = torch.device("cuda:0")
    s = torch.cuda.current_stream().cuda_stream
    # two different shapes back to back: the second call sees the first call's scratch contents
    for (m, n, k, seed) in ((200, 2560, 4096, 90), (130, 257, 2560, 91)):
        w = synth.q8_0(seed, "na", n, k)
        key = "na.%d.%d" % (n, k)
        assert accel.upload_q8_0(key, w, k, n)
        x = torch.from_numpy(synth.normal(seed, "na.x", m, k)).to(dev)
        y_ref = torch.full((m, n), float("nan"), device=dev)
        assert accel.prefill_q8_gemm_dev(key, x.data_ptr(), m, y_ref.data_ptr(), stream=s)
        for call in range(2):
            y = torch.full((m, n), float("nan"), device=dev)
            assert accel.prefill_q8_gemm_noalloc(key, x.data_ptr(), m, y.data_ptr(), stream=s)
            assert accel.device_status(s) == 0
            got, want = y.cpu().numpy(), y_ref.cpu().numpy()
            assert np.isfinite(got).all()
            assert rel_l2(got, want) <= REL_L2_TOL, (m, n, k, call)


def test_noalloc_call_leaves_free_memory_unchanged(accel, synth, pkg):
    """The handle exists (strix_cuda_create has touched the fixed array and the kernels), so a call - even the
    first one with a shape this handle has never seen - must not change the device's free memory."""
    import torch
    dev = torch.device("cuda:0")
    s = torch.cuda.current_stream().cuda_stream
    m, n, k = 77, 300, 1184                                  # never used anywhere else
    assert accel.upload_q8_0("na.fresh", synth.q8_0(93, "nf", n, k), k, n)
    x = torch.from_numpy(synth.normal(93, "nf.x", m, k)).to(dev)
    y = torch.full((m, n), float("nan"), device=dev)
    y_ref = torch.full((m, n), float("nan"), device=dev)
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    assert accel.prefill_q8_gemm_noalloc("na.fresh", x.data_ptr(), m, y.data_ptr(), stream=s)
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0, "the allocation-free entry point changed free device memory by %d bytes" % (free0 - free1)
    assert accel.prefill_q8_gemm_dev("na.fresh", x.data_ptr(), m, y_ref.data_ptr(), stream=s)
    assert rel_l2(y.cpu().numpy(), y_ref.cpu().numpy()) <= REL_L2_TOL


def test_noalloc_refuses_what_does_not_fit(accel, synth, pkg):
    import torch
    dev = torch.device("cuda:0")
    cap = accel.noalloc_scratch_bytes()
    assert cap == 32 << 20
    k, n = 4096, 64
    assert accel.upload_q8_0("na.big", synth.q8_0(92, "nb", n, k), k, n)
    m = cap // k + 1                       # the int8 codes alone exceed the array
    x = torch.zeros(m, k, device=dev)
    y = torch.zeros(m, n, device=dev)
    with pytest.raises(pkg.StrixCudaError) as ei:
        accel.prefill_q8_gemm_noalloc("na.big", x.data_ptr(), m, y.data_ptr())
    assert "scratch" in str(ei.value)
    assert accel.prefill_q8_gemm_noalloc("na.none", x.data_ptr(), 1, y.data_ptr()) is False
