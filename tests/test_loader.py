"""Direct-to-device loading (mynah_b200_model_load): safetensors and GGUF files are mapped and parsed by the library
itself. CPU part: the GGUF files written for the tests are valid for an independent reader (the `gguf` package).
GPU part: a model loaded from a file gives the bits of the same model handed over tensor by tensor."""
import os

import numpy as np
import pytest

import cases


def test_written_gguf_is_readable_by_an_independent_reader(synth, tmp_path):
    gguf = pytest.importorskip("gguf")
    cfg, tensors = cases.build(synth, "rnnt_kq")
    path = str(tmp_path / "model.gguf")
    synth.write_gguf(path, tensors)
    rd = gguf.GGUFReader(path)
    got = {t.name: t for t in rd.tensors}
    assert set(got) == set(tensors)
    for name, t in tensors.items():
        g = got[name]
        assert int(g.tensor_type) == t.ggml_type, name
        assert [int(d) for d in g.shape] == list(reversed(t.shape)), name        # fastest dimension first in the file
        assert np.array_equal(np.asarray(g.data).view(np.uint8).reshape(-1), t.raw), name


@pytest.mark.gpu
@pytest.mark.parametrize("name,ext,quant", [("tdt_q4", ".gguf", 0), ("rnnt_kq", ".gguf", 0), ("ctc_a8", ".safetensors", 1)])
def test_loaded_model_equals_the_tensor_by_tensor_model(gpu_pkg, synth, tmp_path, name, ext, quant):
    a8 = name in cases.A8
    cfg, tensors = cases.build_a8(synth, name) if a8 else cases.build(synth, name)
    wpath, mpath = str(tmp_path / ("model" + ext)), str(tmp_path / "mel_filters.safetensors")
    synth.write_model_file(wpath, tensors)
    synth.write_safetensors(mpath, {"mel_fb": synth.mel_filterbank(cfg.n_mels), "window": synth.hann_window()})
    kw = dict(causal=int(cfg.causal), normalize=cfg.normalize, left=cfg.left, right=cfg.right, blank=cfg.vocab - 1,
              max_symbols=cfg.max_symbols, durations=tuple(cfg.durations), a8=a8)
    a = gpu_pkg.Model.load(wpath, mpath, quant=quant, n_mels=cfg.n_mels, **kw)
    b = cases.device_model(gpu_pkg, synth, cfg, tensors, a8=a8)
    st = a.load_stats()
    assert st["seconds"] > 0 and st["host_bytes"] >= sum(t.raw.size for t in tensors.values())
    audio = synth.synth_audio(1.5, seed=3)
    fa, va = a.log_mel(audio)
    fb, vb = b.log_mel(audio)
    assert va == vb and np.array_equal(fa, fb)
    assert np.array_equal(a.encoder_forward(fa[:va]), b.encoder_forward(fb[:vb]))
    dec = 1 if cfg.decoder == "ctc" else 0
    assert a.transcribe_batch([audio], decoder=dec) == b.transcribe_batch([audio], decoder=dec)
    a.close(); b.close()


@pytest.mark.gpu
def test_loader_errors(gpu_pkg, tmp_path):
    with pytest.raises(gpu_pkg.BackendError, match="cannot open"):
        gpu_pkg.Model.load(str(tmp_path / "missing.gguf"), n_mels=80)
    bad = tmp_path / "bad.gguf"
    bad.write_bytes(b"GGUF" + b"\x09\x00\x00\x00" + b"\x00" * 32)           # unsupported version
    with pytest.raises(gpu_pkg.BackendError, match="version"):
        gpu_pkg.Model.load(str(bad), n_mels=80)
    trunc = tmp_path / "trunc.safetensors"
    trunc.write_bytes((1 << 40).to_bytes(8, "little") + b"{}")              # header longer than the file
    with pytest.raises(gpu_pkg.BackendError, match="header length"):
        gpu_pkg.Model.load(str(trunc), n_mels=80)
