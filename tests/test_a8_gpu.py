"""Int8-activation mode of the encoder (config a8): the ten linears of every layer as integer contractions on the
tensor cores, against outputs of the compiled reference run with its int8 encoder weights and MYNAH_ASR_QGEMM=1
(tests/golden/ref_*_a8.npz, made by tests/golden/make_golden.py in a process with that switch set).

What can be exact is exact: every linear's int32 sums and the float result (float)int32 * ws * sx (tests/test_qmat_gpu.py
checks them bit for bit), and a row's bits do not depend on the batch. What cannot: an activation next to a rounding
boundary goes the other way when the float steps before the quantisation (LayerNorm, softmax, the fp16 K/V of the
attention kernel) differ in their last bits, and one flipped int8 activation is a 1/127 step — two correct
implementations of this mode agree per layer only to about 0.17 sqrt(delta) for float steps that agree to delta.
The tolerances say so: a layer from the reference's own input within 5e-3, the two-layer encoder within 1e-2, both of
the order of the distance between this mode and the float-activation path on the same weights (3e-3 .. 4e-3)."""
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
    assert rel(dm.encoder_layer(0, x), g["layer0"]) < 5e-3
    raw = dm.encoder_forward(f, raw=True)
    assert rel(raw, g["enc_raw"]) < 1e-2
    assert rel(dm.encoder_forward(f), g["enc"]) < 1e-2
    # row stability: a packed batch gives every item the bits it gets alone
    f2, v2 = dm.log_mel(synth.synth_audio(cases.A8_SECONDS[name] * 0.5, seed=8))
    outs = dm.encoder_forward_batch([f, f2[:v2], f[:11]])
    assert rel(outs[0], g["batch0"]) < 1e-2 and rel(outs[1], g["batch1"]) < 1e-2
    assert np.array_equal(outs[0], dm.encoder_forward(f))
    assert np.array_equal(outs[1], dm.encoder_forward(f2[:v2]))
    assert np.array_equal(outs[2], dm.encoder_forward(f[:11]))
    # tokens: teacher-forced on the reference's frames the decoders agree exactly; the whole path equals the
    # decoder run on this path's own frames (the token stream of the reference's run may differ where a frame's
    # top two logits are closer than the two encoders are)
    if cfg.decoder == "ctc":
        assert dm.ctc_decode(g["enc_raw"]) == (g["tokens"].tolist(), g["frames"].tolist())
        res = dm.transcribe_batch([audio], decoder=1)
        assert res[0] == dm.ctc_decode(raw)
    else:
        assert dm.greedy_decode(g["enc"]) == (g["tokens"].tolist(), g["frames"].tolist())
        res = dm.transcribe_batch([audio], decoder=0)
        assert res[0] == dm.greedy_decode(dm.encoder_forward(f))
    same = sum(a == b for a, b in zip(res[0][0], g["tokens"].tolist()))
    print(name, "tokens equal to the reference's int8 run:", same, "of", len(g["tokens"]))
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
