"""Several host threads on one model (the reference's contract: a loaded model is read-only and shared by N threads,
docs/api.md:4-5; its server test tests/test_serve_repro.sh checks that concurrent requests give the text of sequential
ones). Every call takes its own execution context (stream + workspace) over the shared weights, so the calls overlap
on the GPU; each result must have exactly the bits of the same call made alone."""
import threading

import numpy as np
import pytest

import cases

pytestmark = pytest.mark.gpu


def test_concurrent_calls_equal_serial_calls(gpu_pkg, synth):
    cfg, tensors = cases.build(synth, "tdt_q4")
    dm = cases.device_model(gpu_pkg, synth, cfg, tensors)
    dm.set_max_contexts(4)
    audios = [synth.synth_audio(1.0 + 0.37 * i, seed=40 + i) for i in range(8)]
    feats = []
    for a in audios:
        f, v = dm.log_mel(a)
        feats.append(f[:v])
    serial_tok = [dm.transcribe_batch([a, audios[0][:5000]]) for a in audios]
    serial_enc = [dm.encoder_forward(f) for f in feats]
    results, errors = {}, []

    def worker(i):
        try:
            for rep in range(3):                       # several rounds so the threads really overlap
                tok = dm.transcribe_batch([audios[i], audios[0][:5000]])
                enc = dm.encoder_forward(feats[i])
                results[(i, rep)] = (tok, enc)
        except Exception as e:                         # noqa: BLE001 — reported below
            errors.append((i, repr(e)))

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(8)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    for (i, rep), (tok, enc) in results.items():
        assert tok == serial_tok[i], (i, rep)
        assert np.array_equal(enc, serial_enc[i]), (i, rep)
    dm.close()
