"""AED (Canary-style) greedy decoder on the GPU against the compiled reference's outputs
(tests/golden/ref_aed_*.npz, src/decoder_aed.c) and the numpy oracle: token ids must be identical."""
import os

import numpy as np
import pytest

import cases
from oracle import mynah_oracle as O, model_io

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.fixture(scope="module", params=list(cases.AED))
def setup(request, gpu_pkg, synth):
    name = request.param
    cfg, tensors = cases.build(synth, name)
    dm = cases.device_model(gpu_pkg, synth, cfg, tensors, aed_heads=cfg.aed_heads)
    yield name, cfg, tensors, dm, np.load(os.path.join(GOLD, f"ref_{name}.npz"))
    dm.close()


def test_decoder_on_reference_encoder_output(setup):
    name, cfg, tensors, dm, g = setup
    for i in range(2):
        enc = g[f"enc{i}"]
        assert dm.aed_decode(enc, cases.AED_PROMPT, -1, cases.AED_CAP).tolist() == g[f"tokens{i}"].tolist()
        assert dm.aed_decode(enc, cases.AED_PROMPT, int(g[f"eos{i}"]), cases.AED_CAP).tolist() == g[f"tokens_eos{i}"].tolist()
        assert dm.aed_decode(enc, cases.AED_PROMPT[:1], -1, cases.AED_CAP).tolist() == g[f"tokens_start{i}"].tolist()


def test_batch_equals_single_and_oracle(setup):
    """Lock-step batch with different lengths, prompts and budgets == each utterance alone == the oracle."""
    name, cfg, tensors, dm, g = setup
    A = model_io.oracle_model(cfg, tensors)["aed"]
    encs = [g["enc0"], g["enc1"], g["enc0"][:9]]
    prompts = [cases.AED_PROMPT, cases.AED_PROMPT[:2], (3,)]
    caps = [cases.AED_CAP, 11, 1000]                       # the last one runs into the position table's end
    eos = int(g["eos1"])
    got = dm.aed_decode_batch(encs, prompts, eos, caps)
    for e, p, c, t in zip(encs, prompts, caps, got):
        assert list(t) == dm.aed_decode(e, p, eos, c).tolist()
        assert list(t) == O.aed_decode(A, e, p, eos, c).tolist()
    assert any(len(t) for t in got)


def test_edges(setup, gpu_pkg):
    name, cfg, tensors, dm, g = setup
    assert dm.aed_decode(g["enc0"], cases.AED_PROMPT, -1, 0).tolist() == []          # no budget
    with pytest.raises(gpu_pkg.BackendError):
        dm.aed_decode(g["enc0"], (), -1, 4)                                            # no start token
    with pytest.raises(gpu_pkg.BackendError):
        dm.aed_decode(g["enc0"], (cfg.vocab,), -1, 4)                                  # token outside the vocabulary
    long_prompt = tuple(range(1, cfg.aed_max_seq + 5))                                 # prompt longer than the position table
    assert dm.aed_decode(g["enc0"], long_prompt, -1, 4).tolist() == []


def test_whole_path_from_audio(setup, synth):
    """audio -> log-mel -> encoder -> AED decode on the device == the reference's tokens for the same audio."""
    name, cfg, tensors, dm, g = setup
    audios = [synth.synth_audio(2.0, seed=11), synth.synth_audio(1.2, seed=12)]
    delta = cases.AED_CAP - g["enc0"].shape[0]            # budget T + delta == AED_CAP for utterance 0
    out = dm.transcribe_batch_aed(audios, cases.AED_PROMPT, -1, delta)
    assert list(out[0]) == g["tokens0"].tolist()
    A = model_io.oracle_model(cfg, tensors)["aed"]
    cap1 = g["enc1"].shape[0] + delta
    assert list(out[1]) == O.aed_decode(A, g["enc1"], cases.AED_PROMPT, -1, cap1).tolist()
