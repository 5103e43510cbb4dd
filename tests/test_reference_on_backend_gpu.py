"""The reference itself running on this library: its own sources with the two-file patch set of integration/
(an environment selector in backend.c, a quantised-operand hook at the top of mynah_asr_qmat_mul) compiled with its
own -DMYNAH_ASR_CUDA switch and linked against libmynah_b200.so where its cuda_gemm.o stood (`make -C oracle cuda`).
mynah_asr_set_backend("cuda") then has to report the CUDA backend, and the reference's qmat products and encoder
forward — its host code unchanged — have to give what its CPU backend gives (the committed outputs of the unpatched
reference): the drop-in, exercised end to end."""
import os

import numpy as np
import pytest

import cases
from oracle import model_io, ref_binding as R

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def rel(a, b):
    return float(np.linalg.norm(a.astype(np.float64) - b.astype(np.float64)) / max(np.linalg.norm(b), 1e-30))


@pytest.fixture(scope="module")
def patched():
    if not os.path.exists(R.CUDA_LIB_PATH):
        pytest.skip("oracle/_ref/libmynah_ref_cuda.so not built (make -C oracle cuda, where the reference sources are)")
    L = R.cuda_lib()
    yield L
    L.mynah_asr_set_backend(b"cpu")


def test_backend_selection_and_qmat_cases(gpu_pkg, patched):
    assert patched.mynah_asr_set_backend(b"cuda") == 2 and patched.mynah_asr_backend() == 2
    g = np.load(os.path.join(GOLD, "ref_qmat.npz"))          # the cases of the reference's tests/test_qmat.c
    served = 0
    for n, k in ((96, 256), (40, 1024)):
        w = g[f"w_{n}x{k}"]
        for T in (1, 4, 48):
            x = g[f"x_{n}x{k}_T{T}"]
            for q, qn in ((0, "f32"), (1, "q8"), (2, "q4")):
                before = gpu_pkg.launch_count()
                got = R.qmat_mul(w, q, x, library=patched)
                served += gpu_pkg.launch_count() > before
                # the harness frees its weight copy after every call: drop the address-keyed entries, as the
                # reference does for its Metal cache when a model is freed
                gpu_pkg.weights_evict()
                want = g[f"y_{n}x{k}_T{T}_{qn}"]
                assert rel(got, want) < 2e-6, (n, k, T, qn)
    # f32 goes to the device from 24 rows on (the reference's own threshold), the quantised formats for every T
    assert served == 2 * (1 + 3 + 3)
    assert patched.mynah_asr_set_backend(b"cpu") == 0


def test_reference_encoder_forward_on_the_backend(gpu_pkg, synth, patched, tmp_path):
    name = "tdt_q4"
    g = np.load(os.path.join(GOLD, f"ref_{name}.npz"))
    cfg, tensors = cases.build(synth, name)
    wp, mp = model_io.write_reference_files(str(tmp_path), cfg, tensors, synth)
    assert patched.mynah_asr_set_backend(b"cuda") == 2
    rm = R.RefModel(wp, mp, n_mels=cfg.n_mels, normalize=int(cfg.normalize), blank=cfg.vocab - 1, max_symbols=cfg.max_symbols,
                    durations=tuple(cfg.durations), causal=int(cfg.causal), library=patched)
    f = g["feats"][:int(g["valid"])]
    before = gpu_pkg.launch_count()
    enc = rm.encoder_forward(f)
    launches = gpu_pkg.launch_count() - before
    assert launches >= 2 * 10 * cfg.n_layers                   # every large linear of every layer went through the library
    assert rel(enc, g["enc"]) < 1e-5                           # f32-grade: the reference's CPU result
    t, fr = rm.greedy_decode(enc, cfg.max_symbols)
    assert t == g["tokens"].tolist() and fr == g["frames"].tolist()
    # the reference's own int8 mode through the quantised-operand hook
    rq = R.RefModel(wp, mp, quant=1, n_mels=cfg.n_mels, normalize=int(cfg.normalize), blank=cfg.vocab - 1,
                    max_symbols=cfg.max_symbols, durations=tuple(cfg.durations), causal=int(cfg.causal), library=patched)
    enc_q_dev = rq.encoder_forward(f)
    patched.mynah_asr_set_backend(b"cpu")
    enc_q_cpu = rq.encoder_forward(f)
    assert rel(enc_q_dev, enc_q_cpu) < 1e-5
    rq.close()
    rm.close()
    gpu_pkg.weights_evict()
