"""Prompt-conditioned post-encoder MLP (mynah_asr_encoder_post with a prompt id, src/encoder.c:591-614) on the device
against outputs of the compiled reference (tests/golden/ref_rnnt_prompt.npz): single utterance, packed batch with one
prompt id per item, the streaming step, and the greedy tokens of the whole path."""
import os

import numpy as np
import pytest

import cases

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
SECONDS = (1.6, 1.0, 1.3)


def rel(a, b):
    return float(np.linalg.norm(a.astype(np.float64) - b.astype(np.float64)) / max(np.linalg.norm(b), 1e-30))


def test_prompt_mlp(gpu_pkg, synth):
    name = "rnnt_prompt"
    g = np.load(os.path.join(GOLD, f"ref_{name}.npz"))
    cfg, tensors = cases.build(synth, name)
    dm = cases.device_model(gpu_pkg, synth, cfg, tensors)
    audio = [synth.synth_audio(s, seed=21 + i) for i, s in enumerate(SECONDS)]
    feats = []
    for a in audio:
        f, v = dm.log_mel(a)
        feats.append(f[:v])
    for i, pid in enumerate(cases.PROMPT_IDS):
        enc = dm.encoder_forward(feats[i], prompt_id=pid)
        assert rel(enc, g[f"enc{i}"]) < 1e-3
        t, fr = dm.greedy_decode(g[f"enc{i}"])                 # teacher-forced decode of the reference's frames
        assert t == g[f"tokens{i}"].tolist() and fr == g[f"frames{i}"].tolist()
    assert rel(dm.encoder_forward(feats[0]), g["enc0_p0"]) < 1e-3
    # packed batch, one prompt id per item: same bits as each item alone, whatever its neighbours' prompts
    outs = dm.encoder_forward_batch(feats, prompt_ids=cases.PROMPT_IDS)
    for i, pid in enumerate(cases.PROMPT_IDS):
        assert rel(outs[i], g[f"batch{i}"]) < 1e-3
        assert np.array_equal(outs[i], dm.encoder_forward(feats[i], prompt_id=pid))
    with pytest.raises(gpu_pkg.BackendError, match="prompt id"):
        dm.encoder_forward(feats[0], prompt_id=cfg.num_prompts)
    # whole path with prompts: audio in, tokens out
    res = dm.transcribe_batch(audio, prompt_ids=cases.PROMPT_IDS)
    for i in range(3):
        assert res[i][0] == g[f"tokens{i}"].tolist() and res[i][1] == g[f"frames{i}"].tolist()
    # streaming: two streams with different prompts in one lock-step group
    grp = dm.stream_open(2, 6, 0)
    grp.set_prompts([cases.PROMPT_IDS[0], 1])
    mel, pos, outs = feats[0], 0, []
    while pos < mel.shape[0]:
        n = grp.need()
        chunk = mel[pos:pos + n]
        last = pos + n >= mel.shape[0]
        outs.append(grp.step(np.stack([chunk, chunk]), is_last=last))
        pos += n
    got = np.concatenate(outs, axis=1)
    assert rel(got[0], g["stream0"]) < 1e-3
    assert rel(got[1], got[0]) > 1e-2                          # the other stream ran with another prompt
    grp.close()
    dm.close()
