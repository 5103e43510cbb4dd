"""Voice activity and segment planning on the device against outputs of the compiled reference
(tests/golden/ref_vad.npz: mynah_asr_vad_feed / _speech_spans of src/vad.c on the synthetic Silero-shaped model, and the
file-static plan_segments of src/mynah_asr.c reached through oracle/ref_planner.c).

Tolerances: the probabilities within 1e-5 (f32 network, different summation order than the reference's BLAS); spans and
segments identical — they are integer logic over the probabilities and over double-precision window energies formed in
the reference's order."""
import os

import numpy as np
import pytest

import cases

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_vad_spans_and_plans(gpu_pkg, synth):
    g = np.load(os.path.join(GOLD, "ref_vad.npz"))
    cfg, T = synth.make_vad()
    v = gpu_pkg.Vad(cfg["vad"], T)
    for i, (secs, seed) in enumerate(cases.VAD_AUDIO):
        a = synth.speech_like_audio(secs, seed=seed)
        pr = v.probs(a)
        assert pr.shape == g[f"probs{i}"].shape
        assert np.abs(pr - g[f"probs{i}"]).max() < 1e-5
        assert v.speech_spans(a) == [tuple(r) for r in g[f"spans{i}"].tolist()]
        for seg in cases.VAD_SEG_SECONDS:
            assert gpu_pkg.plan_segments(a, 16000, seg) == [tuple(r) for r in g[f"plan_energy{i}_{seg:g}"].tolist()]
            assert gpu_pkg.plan_segments(a, 16000, seg, v) == [tuple(r) for r in g[f"plan_vad{i}_{seg:g}"].tolist()]
        # a signal shorter than the limit is one segment; the planner covers the signal without gaps or overlaps
        assert gpu_pkg.plan_segments(a, 16000, 300.0) == [(0, len(a))]
        plan = gpu_pkg.plan_segments(a, 16000, 5.0)
        assert plan[0][0] == 0 and sum(l for _, l in plan) == len(a) and all(o2 == o1 + l1 for (o1, l1), (o2, _) in zip(plan, plan[1:]))
    quiet = np.zeros(16000, np.float32)
    assert v.speech_spans(quiet) == [] and g["spans_quiet"].shape[0] == 0
    assert gpu_pkg.plan_segments(quiet, 16000, 5.0, v) == [tuple(r) for r in g["plan_quiet"].tolist()]
    assert gpu_pkg.plan_segments(np.zeros(0, np.float32), 16000, 5.0) == [(0, 0)]
    tail = synth.speech_like_audio(1.0, seed=5)[:700]                       # a partial last frame is zero-padded
    assert v.probs(tail).shape == (2,)
    v.close()


def test_vad_rejects_a_contradictory_geometry(gpu_pkg, synth):
    cfg, T = synth.make_vad()
    bad = dict(cfg["vad"])
    bad["encoder_strides"] = [1, 1, 1, 1]                                   # the encoder no longer collapses to one step
    with pytest.raises(gpu_pkg.BackendError):
        gpu_pkg.Vad(bad, T)
