"""CTC forced alignment on the device (mynah_b200_align_ctc) against outputs of the compiled reference
(tests/golden/ref_align.npz) and the reference's own known-answer cases (tests/test_align.c): identical frame runs,
ties included, and the same refusals."""
import os

import numpy as np
import pytest

import cases
from oracle import mynah_oracle as O, model_io

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_known_answers(gpu_pkg):
    V, B = 5, 4

    def peaked(want, peak=10.0):
        s = np.zeros((len(want), V), np.float32)
        s[np.arange(len(want)), want] = peak
        return s
    A = gpu_pkg.align_ctc
    assert A(peaked([B, B, 0, 0, B, B, 1, 2, 2]), [0, 1, 2], B) == (0, [2, 6, 7], [3, 6, 8])
    assert gpu_pkg.align_min_frames([1, 1]) == 3 and gpu_pkg.align_min_frames([0, 1]) == 2
    assert A(peaked([1, B, 1]), [1, 1], B) == (0, [0, 2], [0, 2])
    assert A(peaked([1, B, 1])[:2], [1, 1], B)[0] == -1                       # "a a" cannot fit 2 frames
    assert A(peaked([1, 1, B]), [1, 1], B) == (0, [0, 2], [0, 2])             # the illegal skip is not taken
    assert A(peaked([0, 1]), [0, 1], B) == (0, [0, 1], [0, 1])
    assert A(peaked([B, 3, 3, 3, 3, 3, B]), [3], B) == (0, [1], [5])
    assert A(peaked([0, 1]), [0, B], B)[0] == -1                              # a blank among the labels
    assert A(peaked([0, 1]), [0, 7], B)[0] == -1                              # a label outside the vocabulary


def test_against_reference_outputs(gpu_pkg):
    g = np.load(os.path.join(GOLD, "ref_align.npz"))
    for i, (sc, toks, blank) in enumerate(cases.align_cases()):
        rc, t0, t1 = gpu_pkg.align_ctc(sc, toks, blank)
        assert rc == int(g[f"rc{i}"]), i
        if rc == 0:
            assert t0 == g[f"t0_{i}"].tolist() and t1 == g[f"t1_{i}"].tolist(), i


def test_alignment_from_the_resident_ctc_head(gpu_pkg, synth):
    """The aligner step with the scores kept on the device: the tokens the CTC decoder emitted are aligned back onto
    the frames; every run contains the frame the greedy decoder reported for its token."""
    cfg, tensors = cases.build(synth, "ctc_q8")
    dm = cases.device_model(gpu_pkg, synth, cfg, tensors)
    feats, valid = dm.log_mel(synth.synth_audio(2.5, seed=7))
    raw = dm.encoder_forward(feats[:valid], raw=True)
    toks, frames = dm.ctc_decode(raw)
    t0, t1 = dm.ctc_align(raw, toks)
    M = model_io.oracle_model(cfg, tensors)
    logits = O.gemm_wt(raw, M["ctc_w"]) + M["ctc_b"][None, :]
    rc, r0, r1 = O.align_ctc(logits, toks, cfg.vocab - 1)
    assert rc == 0 and (t0, t1) == (r0, r1)
    assert all(a <= f <= b for a, f, b in zip(t0, frames, t1))
    dm.close()
