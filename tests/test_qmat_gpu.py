"""Quantised matmul on the GPU against the oracle: every stored format, the
bandwidth-bound small-T kernel (T <= 16) and the tensor-core kernel (larger T),
through the C ABI (mynah_b200_qmat_*)."""
import os

import numpy as np
import pytest

from oracle import mynah_oracle as O

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def rel(a, b):
    return float(np.linalg.norm(a.astype(np.float64) - b.astype(np.float64)) / max(np.linalg.norm(b), 1e-30))


def make(pkg, synth, fmt_name, n, k, seed=0, scale=0.02):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((n, k)) * scale).astype(np.float32)
    if fmt_name == "f32":
        return pkg.QMat(pkg.F32, w, n, k), w
    if fmt_name == "mq8":
        q, s = O.quantize_int8(w)
        return pkg.QMat(pkg.MYNAH_Q8, q, n, k, scales=s), O.dequant_int8(q, s)
    if fmt_name == "mq4":
        q, s = O.quantize_int4(w)
        return pkg.QMat(pkg.MYNAH_Q4, q, n, k, scales=s), O.dequant_int4(q, s)
    gt = synth.GGML_NAMES[fmt_name]
    raw = synth.QUANTIZERS[gt](w)
    fmt = {2: pkg.GGML_Q4_0, 8: pkg.GGML_Q8_0, 12: pkg.GGML_Q4_K, 14: pkg.GGML_Q6_K}[gt]
    return pkg.QMat(fmt, raw, n, k), O.ggml_dequant(gt, raw).reshape(n, k)


FORMATS = ["f32", "q8_0", "q4_0", "q4_k", "q6_k", "mq8", "mq4"]


@pytest.mark.parametrize("name,gtype", [("Q8_0", 8), ("Q4_0", 2), ("Q4_K", 12), ("Q6_K", 14)])
def test_device_block_decode_known_answers(gpu_pkg, name, gtype):
    """The device decoders against the reference's llama.cpp-generated vectors, bit for bit."""
    raw = np.fromfile(os.path.join(GOLD, "ingot", name + ".bin"), np.uint8)
    ref = np.fromfile(os.path.join(GOLD, "ingot", name + ".ref"), np.float32)
    fmt = {2: gpu_pkg.GGML_Q4_0, 8: gpu_pkg.GGML_Q8_0, 12: gpu_pkg.GGML_Q4_K, 14: gpu_pkg.GGML_Q6_K}[gtype]
    k = 256
    n = ref.size // k
    q = gpu_pkg.QMat(fmt, raw, n, k)
    assert np.array_equal(q.dequant().reshape(-1).view(np.uint32), ref.view(np.uint32))
    # and through the small-T kernel: a one-hot activation reads a weight column exactly
    x = np.zeros((2, k), np.float32); x[0, 5] = 1.0; x[1, 200] = 1.0
    y = q.mul(x)
    assert np.array_equal(y[0], ref.reshape(n, k)[:, 5]) and np.array_equal(y[1], ref.reshape(n, k)[:, 200])


@pytest.mark.parametrize("fmt", FORMATS)
@pytest.mark.parametrize("T", [1, 2, 3, 4, 7, 16])
def test_small_T_streams_stored_blocks(gpu_pkg, synth, fmt, T):
    for n, k in ((200, 1024), (67, 256), (130, 4096), (37, 768)):
        if fmt in ("q4_k", "q6_k") and k % 256:
            continue
        q, wd = make(gpu_pkg, synth, fmt, n, k, seed=n + T)
        x = np.random.default_rng(T).standard_normal((T, k)).astype(np.float32)
        ref = x.astype(np.float64) @ wd.astype(np.float64).T
        assert rel(q.mul(x), ref) < 3e-6, (fmt, n, k)
        # Q4_0 / Q8_0 / Q4_K default to the tcgen05 streaming kernel (T <= 8); the warp-level tensor-core
        # kernel (Q4_0 / Q8_0) and the scalar one must agree
        assert rel(q.mul(x, gpu_pkg.MMA_SYNC), ref) < 3e-6, (fmt, n, k)
        assert rel(q.mul(x, gpu_pkg.SCALAR), ref) < 2e-6, (fmt, n, k)
        q.close()


@pytest.mark.parametrize("fmt", ["q4_0", "q8_0", "q4_k"])
def test_streaming_kernel_work_splits(gpu_pkg, synth, fmt):
    """Shapes that drive the tcgen05 streaming kernel through each of its work splits: several row
    tiles per CTA (more tiles than multiprocessors), one K slice, many K slices, K beyond what one
    CTA holds (8192) with many tiles, and long runs of stages per CTA at every read-back width; ragged last tile everywhere."""
    shapes = ((20001, 256, (1, 5)), (19001, 128, (2,)), (300, 8192, (1, 8)), (9700, 8192, (1,)), (19000, 4096, (4, 8)), (129, 1024, (3,)))
    if fmt == "q4_k":       # 256-element super-blocks; smaller matrices (the numpy K-quantiser is slow)
        shapes = ((20001, 256, (1, 5)), (300, 8192, (1, 8)), (2500, 8192, (2,)), (19000, 1024, (4, 8)), (129, 1024, (3,)))
    for n, k, Ts in shapes:
        q, wd = make(gpu_pkg, synth, fmt, n, k, seed=n)
        for T in Ts:
            x = np.random.default_rng(T).standard_normal((T, k)).astype(np.float32)
            ref = x.astype(np.float64) @ wd.astype(np.float64).T
            y = q.mul(x)
            assert rel(y, ref) < 3e-6, (fmt, n, k, T)
            assert np.array_equal(y, q.mul(x)), "two runs differ"
        q.close()


@pytest.mark.parametrize("fmt", FORMATS)
def test_large_T_tensor_core_path(gpu_pkg, synth, fmt):
    for T, n, k in ((17, 96, 256), (48, 200, 1024), (300, 1030, 512), (129, 8198, 640)):
        if fmt in ("q4_k", "q6_k") and k % 256:
            continue
        q, wd = make(gpu_pkg, synth, fmt, n, k, seed=T)
        x = np.random.default_rng(T).standard_normal((T, k)).astype(np.float32)
        ref = x.astype(np.float64) @ wd.astype(np.float64).T
        # 3-term split: f32 grade. The tensor core truncates when it aligns addends, so a sum of
        # same-sign terms (the T=48 case: x is correlated with W) drifts a few 1e-6; random signs ~1e-6.
        assert rel(q.mul(x), ref) < 2e-5, (fmt, T, n, k)
        assert rel(O.gemm_wt(x, wd), ref) < 3e-6                    # (the f32 sgemm itself, for scale)
        assert rel(q.mul(x, gpu_pkg.FAST), ref) < 1e-3, (fmt, T, n, k)   # single fp16 pass
        q.close()


def test_edge_shapes(gpu_pkg, synth):
    q, wd = make(gpu_pkg, synth, "q8_0", 5, 64)
    for T in (1, 16, 17, 127, 128, 129):
        x = np.random.default_rng(T).standard_normal((T, 64)).astype(np.float32)
        assert rel(q.mul(x), O.gemm_wt(x, wd)) < 5e-6
    assert q.mul(np.zeros((0, 64), np.float32)).shape == (0, 5)          # empty input
    z = q.mul(np.zeros((3, 64), np.float32))
    assert np.array_equal(z, np.zeros((3, 5), np.float32))
    q.close()
    with pytest.raises(gpu_pkg.BackendError):                             # k not a block multiple
        gpu_pkg.QMat(gpu_pkg.GGML_Q4_K, np.zeros(144, np.uint8), 1, 200)


def test_row_stability(gpu_pkg, synth):
    """A row's output bits do not depend on what else is in the batch, nor on where
    the row sits in it (the property the reference states for its packed GEMMs,
    tests/test_batch.c:1-3), within each kernel family."""
    q, _ = make(gpu_pkg, synth, "q4_0", 512, 1024)
    rng = np.random.default_rng(9)
    x = rng.standard_normal((300, 1024)).astype(np.float32)
    full = q.mul(x)
    sub = q.mul(x[40:200])
    assert np.array_equal(full[40:200], sub)
    perm = rng.permutation(300)
    assert np.array_equal(q.mul(x[perm]), full[perm])
    assert np.array_equal(q.mul(x[100:117]), full[100:117])               # 17 rows: still the tensor-core path
    small = q.mul(x[:16])
    assert np.array_equal(q.mul(x[3:9]), small[3:9])                      # small-T kernel: same property
    q.close()


@pytest.mark.parametrize("fmt", ["f32", "q8_0", "q4_k"])
def test_few_rows_kernel(gpu_pkg, synth, fmt):
    """The decoder-position contraction (weights on the 128-row side of the MMA, K slices over the CTAs of a cluster,
    slice sums added in slice order): f32-grade against the f64 product at every row count and at shapes with 1, 2, 4
    and 8 slices, ragged weight-row tiles included; a row's bits depend neither on the number of rows in the launch (so
    neither on the 32 / 64 / 128-wide variant nor on the 128-row grouping) nor on its place among them."""
    FR = gpu_pkg.FEW_ROWS
    for n, k in ((300, 256), (1024, 1024), (4096 + 40, 512), (136, 4096), (16384, 256)):
        q, wd = make(gpu_pkg, synth, fmt, n, k, seed=n + k)
        rng = np.random.default_rng(n)
        x = rng.standard_normal((200, k)).astype(np.float32)
        ref = x.astype(np.float64) @ wd.astype(np.float64).T
        full = q.mul(x, FR)                                             # 128 + 72 rows: two groups
        assert rel(full, ref) < 2e-5, (fmt, n, k)
        for T in (1, 2, 31, 32, 33, 64, 65, 128, 129):
            assert np.array_equal(q.mul(x[:T], FR), full[:T]), (fmt, n, k, T)
        assert np.array_equal(q.mul(x[150:181], FR), full[150:181])
        perm = rng.permutation(200)
        assert np.array_equal(q.mul(x[perm], FR), full[perm])
        assert rel(q.mul(x[:40], FR | gpu_pkg.FAST), ref[:40]) < 1e-3   # single fp16 product
        assert rel(full, q.mul(x)) < 1e-5                               # and next to the many-row kernel on the same planes
        q.close()


def test_a8_block_dots_bit_exact(gpu_pkg, synth):
    """int8 activations: the int32 dot of every 32-element block is exact
    (quantize_act_int8 + dot kernels, src/qmat.c:186-202,285-364)."""
    rng = np.random.default_rng(5)
    n, k, T = 48, 512, 5
    w = rng.uniform(-1, 1, (n, k)).astype(np.float32)
    x = rng.uniform(-1, 1, (T, k)).astype(np.float32)
    qx, sx = O.quantize_act_int8(x)
    # reference-native int8 (per-row scale)
    q8, s8 = O.quantize_int8(w)
    m = gpu_pkg.QMat(gpu_pkg.MYNAH_Q8, q8, n, k, scales=s8)
    dots, sxd, out = m.block_dots(x)
    want = (qx.astype(np.int32).reshape(T, 1, k // 32, 32) * q8.astype(np.int32).reshape(1, n, k // 32, 32)).sum(3)
    assert np.array_equal(dots, want) and np.array_equal(sxd, sx)
    assert np.array_equal(out, O.qmat_mul_a8_q8(x, q8, s8))               # (float)int32 * ws * sx, bit for bit
    assert np.array_equal(m.mul(x, gpu_pkg.A8), out)
    m.close()
    # reference-native int4 (group scales)
    q4, s4 = O.quantize_int4(w)
    m = gpu_pkg.QMat(gpu_pkg.MYNAH_Q4, q4, n, k, scales=s4)
    dots, _, out = m.block_dots(x)
    assert np.array_equal(dots, O.int_dots_q4(qx, O.unpack_int4(q4)))
    assert rel(out, O.qmat_mul_a8_q4(x, q4, s4)) < 1e-6
    m.close()
    # ggml Q8_0 / Q4_0 blocks: integer parts of the stored blocks
    for name, gt, fmt in (("q8_0", 8, gpu_pkg.GGML_Q8_0), ("q4_0", 2, gpu_pkg.GGML_Q4_0)):
        raw = synth.QUANTIZERS[gt](w * 0.02)
        m = gpu_pkg.QMat(fmt, raw, n, k)
        dots, _, out = m.block_dots(x)
        if gt == 8:
            qi = raw.reshape(-1, 34)[:, 2:].view(np.int8).astype(np.int32).reshape(n, k // 32, 32)
            d = raw.reshape(-1, 34)[:, :2].copy().view(np.float16).astype(np.float32).reshape(n, k // 32)
        else:
            b = raw.reshape(-1, 18)[:, 2:]
            qi = np.concatenate([(b & 15).astype(np.int32) - 8, (b >> 4).astype(np.int32) - 8], 1).reshape(n, k // 32, 32)
            d = raw.reshape(-1, 18)[:, :2].copy().view(np.float16).astype(np.float32).reshape(n, k // 32)
        want = (qx.astype(np.int32).reshape(T, 1, k // 32, 32) * qi[None]).sum(3)
        assert np.array_equal(dots, want)
        ref = (want.astype(np.float64) * d[None].astype(np.float64)).sum(2) * sx[:, None].astype(np.float64)
        assert rel(out, ref) < 1e-6
        m.close()


def test_against_reference_qmat_outputs(gpu_pkg):
    """The cases of the reference's tests/test_qmat.c, against outputs of the compiled
    reference (tests/golden/ref_qmat.npz)."""
    g = np.load(os.path.join(GOLD, "ref_qmat.npz"))
    for n, k in ((96, 256), (40, 1024)):
        w = g[f"w_{n}x{k}"]
        q8, s8 = O.quantize_int8(w)
        q4, s4 = O.quantize_int4(w)
        mf = gpu_pkg.QMat(gpu_pkg.F32, w, n, k)
        m8 = gpu_pkg.QMat(gpu_pkg.MYNAH_Q8, q8, n, k, scales=s8)
        m4 = gpu_pkg.QMat(gpu_pkg.MYNAH_Q4, q4, n, k, scales=s4)
        for T in (1, 4, 48):
            x = g[f"x_{n}x{k}_T{T}"]
            assert rel(mf.mul(x), g[f"y_{n}x{k}_T{T}_f32"]) < 5e-6
            if T <= 16:    # the reference runs int8 activations here
                assert rel(m8.mul(x, gpu_pkg.A8), g[f"y_{n}x{k}_T{T}_q8"]) < 3e-7
                assert rel(m4.mul(x, gpu_pkg.A8), g[f"y_{n}x{k}_T{T}_q4"]) < 1e-6
            else:          # and dequant + sgemm here
                assert rel(m8.mul(x), g[f"y_{n}x{k}_T{T}_q8"]) < 5e-6
                assert rel(m4.mul(x), g[f"y_{n}x{k}_T{T}_q4"]) < 5e-6
        assert rel(gpu_pkg.gemm_wt(g[f"x_{n}x{k}_T48"], w), g[f"y_{n}x{k}_T48_f32"]) < 5e-6
        for m in (mf, m8, m4):
            m.close()


def test_address_keyed_hooks(gpu_pkg, synth):
    """mynah_asr_cuda_gemm_wt under the reference's own name and mynah_b200_qgemm: a weight is uploaded on the
    first call with its host address, found by address afterwards, and dropped by the evict call."""
    pkg = gpu_pkg
    pkg.weights_evict()
    rng = np.random.default_rng(3)
    w = (rng.standard_normal((96, 256)) * 0.05).astype(np.float32)
    for T in (1, 5, 40):
        x = rng.standard_normal((T, 256)).astype(np.float32)
        assert rel(pkg.cuda_gemm_wt(x, w), x.astype(np.float64) @ w.astype(np.float64).T) < 3e-6
    assert pkg.weights_resident() == 1
    raw = synth.QUANTIZERS[2](w)                       # Q4_0 blocks of the same matrix
    wd = O.ggml_dequant(2, raw).reshape(96, 256)
    x = rng.standard_normal((3, 256)).astype(np.float32)
    y = pkg.qgemm(raw, pkg.GGML_Q4_0, 96, 256, x)
    assert rel(y, x.astype(np.float64) @ wd.astype(np.float64).T) < 3e-6
    assert np.array_equal(y, pkg.qgemm(raw, pkg.GGML_Q4_0, 96, 256, x))
    h = pkg.QMat(pkg.GGML_Q4_0, raw, 96, 256)
    assert np.array_equal(y, h.mul(x))                 # the same bits as through a handle
    h.close()
    assert pkg.weights_resident() == 2
    pkg.weights_evict()
    assert pkg.weights_resident() == 0


def test_values_outside_the_fp16_operand_range_are_reported(gpu_pkg):
    """The tensor-core path carries operands as fp16 (hi, lo) pairs, which end at 65504. A larger activation or
    weight must not come back as a silent inf/NaN: the call fails (-1), so a host using the reference's hook
    convention falls back to its CPU path. Just below the limit the product is still f32-grade."""
    rng = np.random.default_rng(5)
    n, k, T = 64, 256, 40                                   # T > 16: the contraction kernel
    w = rng.uniform(-1, 1, (n, k)).astype(np.float32)
    x = rng.uniform(-1, 1, (T, k)).astype(np.float32)
    m = gpu_pkg.QMat(gpu_pkg.F32, w, n, k)
    big = (x * 6.0e4).astype(np.float32)                    # |x| < 65504
    want = big.astype(np.float64) @ w.astype(np.float64).T
    assert np.abs(m.mul(big) - want).max() <= 2e-6 * np.abs(want).max()
    bad = x.copy()
    bad[3, 7] = 1.0e5
    with pytest.raises(gpu_pkg.BackendError, match="65504"):
        m.mul(bad)
    assert np.abs(m.mul(x) - x.astype(np.float64) @ w.astype(np.float64).T).max() <= 1e-4     # the handle still works
    m.close()
    wbad = w.copy()
    wbad[0, 0] = 7.0e4
    mb = gpu_pkg.QMat(gpu_pkg.F32, wbad, n, k)              # the handle exists (stored values, small-T products) ...
    want4 = x[:4].astype(np.float64) @ wbad.astype(np.float64).T
    assert np.abs(mb.mul(x[:4]) - want4).max() <= 1e-5 * np.abs(want4).max()
    with pytest.raises(gpu_pkg.BackendError, match="65504"):
        mb.mul(x)                                           # ... but the many-row tensor-core product refuses
    mb.close()
    # the reference's hook under its own name returns -1 (the caller's cue to fall back)
    wk = np.ascontiguousarray(w)
    with pytest.raises(gpu_pkg.BackendError):
        gpu_pkg.cuda_gemm_wt(bad, wk)
    gpu_pkg.weights_evict()


def test_a8_many_rows_on_the_tensor_cores_bit_exact(gpu_pkg):
    """Int8 activations x reference-native int8 weights for more than 16 rows (tcgen05 kind::i8 contraction): the
    result is (float)int32 * ws * sx with the exact int32 dot, so it equals the CPU restatement bit for bit, and a
    row's bits do not depend on how many rows are multiplied with it (the reference's MYNAH_ASR_QGEMM=1 arithmetic,
    src/qmat.c:598-643)."""
    rng = np.random.default_rng(17)
    for n, k in ((384, 1024), (200, 256), (1025, 512)):
        w = rng.uniform(-1, 1, (n, k)).astype(np.float32)
        q8, s8 = O.quantize_int8(w)
        m = gpu_pkg.QMat(gpu_pkg.MYNAH_Q8, q8, n, k, scales=s8)
        x = (rng.standard_normal((300, k)) * rng.uniform(0.1, 30, (300, 1))).astype(np.float32)
        x[5] = 0.0                                              # an all-zero row: scale 0, output 0
        want = O.qmat_mul_a8_q8(x, q8, s8)
        got = m.mul(x, gpu_pkg.A8)
        assert np.array_equal(got, want), (n, k)
        for T in (17, 129):                                     # fewer rows, other tile counts: same bits per row
            assert np.array_equal(m.mul(x[:T], gpu_pkg.A8), want[:T]), (n, k, T)
        assert np.array_equal(m.mul(x[:9], gpu_pkg.A8), want[:9])          # the row-dot kernel below 17 rows agrees too
        m.close()
