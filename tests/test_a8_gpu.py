"""Int8-activation mode of the encoder (config a8): the ten linears of every layer as integer contractions on the
tensor cores, against outputs of the compiled reference run with its int8 encoder weights and MYNAH_ASR_QGEMM=1
(tests/golden/ref_*_a8.npz, made by tests/golden/make_golden.py in a process with that switch set).

Tolerances: one layer from the reference's own input agrees to 1e-4 (the integer sums are exact; the float steps
around them agree to ~1e-6); the whole encoder to the stated 1e-3 — a value next to a rounding boundary may go the
other way after float steps that differ in the last bits, and one flipped int8 activation is a 1/127 step."""
import os

import numpy as np
import pytest

import cases
from oracle import mynah_oracle as O, model_io

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def rel(a, b):
    return float(np.linalg.norm(a.astype(np.float64) - b.astype(np.float64)) / max(np.linalg.norm(b), 1e-30))


@pytest.mark.parametrize("name", list(cases.A8))
def test_int8_activation_encoder(gpu_pkg, synth, name):
    g = np.load(os.path.join(GOLD, f"ref_{name}.npz"))
    cfg, tensors = cases.build_a8(synth, name)
    dm = cases.device_model(gpu_pkg, synth, cfg, tensors, a8=True)
    audio = synth.synth_audio(cases.A8_SECONDS[name], seed=7)
    feats, valid = dm.log_mel(audio)
    f = feats[:valid]
    x = dm.subsampling_forward(f)
    assert rel(dm.encoder_layer(0, x), g["layer0"]) < 1e-4
    raw = dm.encoder_forward(f, raw=True)
    assert rel(raw, g["enc_raw"]) < 1e-3
    assert rel(dm.encoder_forward(f), g["enc"]) < 1e-3
    # row stability: a packed batch gives every item the bits it gets alone
    f2, v2 = dm.log_mel(synth.synth_audio(cases.A8_SECONDS[name] * 0.5, seed=8))
    outs = dm.encoder_forward_batch([f, f2[:v2], f[:11]])
    assert rel(outs[0], g["batch0"]) < 1e-3 and rel(outs[1], g["batch1"]) < 1e-3
    assert np.array_equal(outs[0], dm.encoder_forward(f))
    assert np.array_equal(outs[1], dm.encoder_forward(f2[:v2]))
    assert np.array_equal(outs[2], dm.encoder_forward(f[:11]))
    # tokens: teacher-forced on the reference's frames, and the whole path
    if cfg.decoder == "ctc":
        assert dm.ctc_decode(g["enc_raw"]) == (g["tokens"].tolist(), g["frames"].tolist())
        res = dm.transcribe_batch([audio], decoder=1)
    else:
        assert dm.greedy_decode(g["enc"]) == (g["tokens"].tolist(), g["frames"].tolist())
        res = dm.transcribe_batch([audio], decoder=0)
    assert res[0][0] == g["tokens"].tolist() and res[0][1] == g["frames"].tolist()
    dm.close()
    # the same weights with float activations are a different (and also valid) path: the reference's default
    a16 = cases.device_model(gpu_pkg, synth, cfg, tensors)
    r16 = a16.encoder_forward(f, raw=True)
    assert rel(r16, g["enc_raw_f32"]) < 1e-3 and rel(r16, g["enc_raw"]) > 2e-3
    a16.close()


def test_int8_activation_mode_needs_native_int8_weights(gpu_pkg, synth):
    cfg, tensors = cases.build(synth, "ctc_q8")
    with pytest.raises(gpu_pkg.BackendError, match="a8 mode"):
        cases.device_model(gpu_pkg, synth, cfg, tensors, a8=True)
