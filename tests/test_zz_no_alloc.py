"""The allocation-free A8 entry point (mynah_b200_qmat_mul_a8_static) against the
regular one (mynah_b200_qmat_mul with the A8 flag), through the C ABI.

Who needs it: a host that must not allocate device memory once it is serving — a
streaming thread fed in real time (cudaMalloc/cudaFree stall every stream of the
process for an unbounded time) or a process whose GPU memory is budgeted up front.
Such a caller owns its input and output buffers on the device and the library keeps
its only scratch (int8 activations + their scales) in a fixed built-in array.

Collected last on purpose (file name), so a run that stops at the first failure has
already gone through every other test. Works alone in a fresh process and after the
rest of the suite: it shares no state with the other tests but the library itself.
"""
import numpy as np
import pytest

from oracle import mynah_oracle as O

pytestmark = pytest.mark.gpu


def _device_buffers(torch, x, n):
    xd = torch.from_numpy(x).cuda()
    od = torch.empty((x.shape[0], n), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()          # the library runs on its own stream
    return xd, od


def test_static_scratch_matches_regular_entry_point(gpu_pkg, synth):
    torch = pytest.importorskip("torch")
    rng = np.random.default_rng(21)
    n, k = 192, 1024
    w = rng.uniform(-1, 1, (n, k)).astype(np.float32)
    q8, s8 = O.quantize_int8(w)
    raw40 = synth.QUANTIZERS[synth.GGML_Q4_0](w * 0.02)
    cases = [(gpu_pkg.QMat(gpu_pkg.MYNAH_Q8, q8, n, k, scales=s8), "native int8"),
             (gpu_pkg.QMat(gpu_pkg.GGML_Q4_0, raw40, n, k), "ggml Q4_0")]
    for m, what in cases:
        # two calls in a row with different row counts: the shared scratch keeps the first
        # call's contents, the second must not be affected by them
        for T in (16, 3):
            x = rng.uniform(-1, 1, (T, k)).astype(np.float32)
            want = m.mul(x, gpu_pkg.A8)                        # existing entry point (allocates its scratch)
            xd, od = _device_buffers(torch, x, n)
            m.mul_a8_static(xd.data_ptr(), od.data_ptr(), T)
            got = od.cpu().numpy()
            assert np.array_equal(got, want), what             # same kernels, same bits
            if what == "native int8":
                # the native format has a bit-exact CPU restatement: (float)int32 * ws * sx
                assert np.array_equal(got, O.qmat_mul_a8_q8(x, q8, s8)), "native int8 against the oracle"
        m.close()


def test_static_scratch_limits(gpu_pkg):
    torch = pytest.importorskip("torch")
    n, k = 8, 64
    m = gpu_pkg.QMat(gpu_pkg.MYNAH_Q8, np.ones((n, k), np.int8), n, k, scales=np.ones(n, np.float32))
    x = np.ones((17, k), np.float32)
    xd, od = _device_buffers(torch, x, n)
    with pytest.raises(gpu_pkg.BackendError, match="exceed"):  # more rows than the built-in scratch holds
        m.mul_a8_static(xd.data_ptr(), od.data_ptr(), 17)
    m.mul_a8_static(xd.data_ptr(), od.data_ptr(), 0)           # empty call is a no-op
    m.close()
    big = gpu_pkg.QMat(gpu_pkg.MYNAH_Q8, np.ones((2, 16384), np.int8), 2, 16384, scales=np.ones(2, np.float32))
    xb = np.ones((1, 16384), np.float32)
    xd, od = _device_buffers(torch, xb, 2)
    with pytest.raises(gpu_pkg.BackendError, match="exceed"):  # k beyond the limit
        big.mul_a8_static(xd.data_ptr(), od.data_ptr(), 1)
    big.close()
    # a format without an int8-activation mode is refused before anything is launched
    f32 = gpu_pkg.QMat(gpu_pkg.F32, np.ones((4, 64), np.float32), 4, 64)
    xd, od = _device_buffers(torch, np.ones((2, 64), np.float32), 4)
    with pytest.raises(gpu_pkg.BackendError, match="int8-activation"):
        f32.mul_a8_static(xd.data_ptr(), od.data_ptr(), 2)
    f32.close()
