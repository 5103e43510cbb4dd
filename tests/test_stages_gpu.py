"""Per-stage and whole-path parity of the CUDA path against the oracle and against
outputs of the compiled reference (tests/golden/ref_*.npz), through the C ABI.
Tolerances: the reference's own ladder (tests/test_features.c:64 5e-4 abs on mel,
tests/test_subsampling.c:73 1e-5 x scale, tests/test_encoder.c:19-39 1e-4 x scale per
layer) and the stated bar of relative L2 <= 1e-3 on the encoder output."""
import os

import numpy as np
import pytest

import cases
from oracle import mynah_oracle as O, model_io

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
AUDIO_SECONDS = {"ctc_q8": 2.5, "tdt_q4": 3.0, "rnnt_kq": 2.0, "ctc_bias": 1.5}


def rel(a, b):
    return float(np.linalg.norm(a.astype(np.float64) - b.astype(np.float64)) / max(np.linalg.norm(b), 1e-30))


@pytest.fixture(scope="module", params=list(cases.TINY))
def setup(request, gpu_pkg, synth):
    name = request.param
    cfg, tensors = cases.build(synth, name)
    dm = cases.device_model(gpu_pkg, synth, cfg, tensors)
    g = np.load(os.path.join(GOLD, f"ref_{name}.npz"))
    yield name, cfg, tensors, dm, g
    dm.close()


def test_log_mel(setup, synth):
    name, cfg, _, dm, g = setup
    audio = synth.synth_audio(AUDIO_SECONDS[name], seed=7)
    feats, valid = dm.log_mel(audio)
    assert valid == int(g["valid"]) and feats.shape == g["feats"].shape
    assert np.abs(feats - g["feats"]).max() <= 5e-5
    assert np.all(feats[valid:] == 0)


def test_log_mel_edges(setup, synth):
    _, cfg, _, dm, _ = setup
    for n in (0, 1, 159, 160, 161, 400, 4000):
        a = synth.synth_audio(1.0, seed=n)[:n]
        feats, valid = dm.log_mel(a)
        fo, vo = O.log_mel(a, synth.mel_filterbank(cfg.n_mels), synth.hann_window(),
                           normalize_per_feature=cfg.normalize)
        assert valid == vo and feats.shape == fo.shape
        assert np.abs(feats - fo).max() <= 5e-5 if feats.size else True


def test_subsampling(setup):
    _, cfg, _, dm, g = setup
    f = g["feats"][:int(g["valid"])]
    out = dm.subsampling_forward(f)
    assert out.shape == g["subsampling"].shape
    assert np.abs(out - g["subsampling"]).max() <= 1e-5 * np.abs(g["subsampling"]).max() * 10
    for T in (1, 2, 7, 8, 9, 17):          # ragged lengths around the stride boundaries
        o = dm.subsampling_forward(f[:T])
        ref = O.subsampling_forward(model_io.oracle_model(cfg, setup[2])["ss"], f[:T], cfg.causal)
        assert o.shape == ref.shape and rel(o, ref) < 1e-5


def test_encoder_layer(setup):
    _, cfg, tensors, dm, g = setup
    out = dm.encoder_layer(0, g["subsampling"])
    assert np.abs(out - g["layer0"]).max() <= 1e-4 * np.abs(g["layer0"]).max() * 5
    assert rel(out, g["layer0"]) < 2e-4
    # limited context: chunked window of the streaming-capable models
    M = model_io.oracle_model(cfg, tensors)
    pe = O.pos_emb(g["subsampling"].shape[0], cfg.d_model)
    for left, right in ((8, 1), (6, 0), (4, 3)):
        li = cfg.n_layers - 1
        want = O.encoder_layer(M["layers"][li], g["subsampling"], pe, cfg.n_heads, cfg.causal, left, right)
        assert rel(dm.encoder_layer(li, g["subsampling"], left, right), want) < 2e-4


def test_encoder_forward(setup):
    _, cfg, _, dm, g = setup
    f = g["feats"][:int(g["valid"])]
    assert rel(dm.encoder_forward(f, raw=True), g["enc_raw"]) < 1e-3
    assert rel(dm.encoder_forward(f), g["enc"]) < 1e-3
    assert rel(dm.encoder_forward(f, left=8, right=1, raw=True), g["enc_lim"]) < 1e-3


def test_batch_equals_single_bitwise(setup, synth):
    """Packed batch == one call per item, bit for bit (row stability), and both match
    the reference's packed batch."""
    name, cfg, _, dm, g = setup
    f0 = g["feats"][:int(g["valid"])]
    a2 = synth.synth_audio(AUDIO_SECONDS[name] * 0.6, seed=8)
    f2, v2 = dm.log_mel(a2)
    f2 = f2[:v2]
    outs = dm.encoder_forward_batch([f0, f2, f0[:9]])
    assert rel(outs[0], g["batch0"]) < 1e-3 and rel(outs[1], g["batch1"]) < 1e-3
    assert np.array_equal(outs[0], dm.encoder_forward(f0))
    assert np.array_equal(outs[1], dm.encoder_forward(f2))
    assert np.array_equal(outs[2], dm.encoder_forward(f0[:9]))
    swapped = dm.encoder_forward_batch([f2, f0])
    assert np.array_equal(swapped[0], outs[1]) and np.array_equal(swapped[1], outs[0])


def test_attention_kernels_agree(setup, gpu_pkg, synth):
    """The tiled tensor-core attention against the plain one-warp-per-query kernel."""
    _, cfg, tensors, dm, g = setup
    plain = cases.device_model(gpu_pkg, synth, cfg, tensors, attn_impl=1)
    a = dm.encoder_layer(0, g["subsampling"])
    b = plain.encoder_layer(0, g["subsampling"])
    assert rel(a, b) < 1e-4
    plain.close()


def test_decoders_on_reference_encoder_output(setup):
    """Teacher-forced: the reference's encoder output through the device decoder."""
    _, cfg, _, dm, g = setup
    if cfg.decoder == "ctc":
        t, f = dm.ctc_decode(g["enc_raw"])
    else:
        t, f = dm.greedy_decode(g["enc"])
    assert t == g["tokens"].tolist()
    assert f == g["frames"].tolist()


def test_whole_path_tokens(setup, synth):
    """Audio in, tokens out, everything resident: identical greedy tokens and frames."""
    name, cfg, _, dm, g = setup
    audio = synth.synth_audio(AUDIO_SECONDS[name], seed=7)
    dec = 1 if cfg.decoder == "ctc" else 0
    res = dm.transcribe_batch([audio, audio[: len(audio) // 2], audio], decoder=dec)
    assert res[0][0] == g["tokens"].tolist() and res[0][1] == g["frames"].tolist()
    assert res[2] == res[0]
    empty = dm.transcribe_batch([audio[:0], audio], decoder=dec)       # empty item in a batch
    assert empty[0] == ([], []) and empty[1] == res[0]


def test_fast_mode_within_tolerance(setup, gpu_pkg, synth):
    """Single fp16 product per term (the extra `fast` key of the benchmark), held to the stated bar of relative L2 1e-3
    against the compiled reference — the same bound the full-size models are held to in test_config_shapes_gpu.py —
    and switchable at run time on one model: back in strict mode the bits are those of a model built strict."""
    name, cfg, tensors, dm, g = setup
    fast = cases.device_model(gpu_pkg, synth, cfg, tensors, strict=False)
    f = g["feats"][:int(g["valid"])]
    e = rel(fast.encoder_forward(f, raw=True), g["enc_raw"])
    print(name, "fast-mode encoder rel-L2", e)
    assert e < 1e-3
    strict_out = dm.encoder_forward(f, raw=True)
    dm.set_strict(False)
    assert np.array_equal(dm.encoder_forward(f, raw=True), fast.encoder_forward(f, raw=True))
    dm.set_strict(True)
    assert np.array_equal(dm.encoder_forward(f, raw=True), strict_out)
    fast.close()


def test_tcgen05_attention_long_segments(gpu_pkg, synth):
    """Full attention over 128-wide heads runs on the tcgen05 kernel (128-query tiles, 64-key tiles, rk ring):
    against the plain kernel, the warp-level tiled kernel and the oracle, over lengths that exercise one and
    several query / key tiles, ragged last tiles and the ring wrap; and in a packed batch."""
    cfg = synth.config("attn128", d_model=256, n_layers=1, n_heads=2, ffn_dim=256, n_mels=80, decoder="ctc", vocab=33,
                       wtype="q8_0")
    tensors = synth.make_model(cfg, seed=5)
    tc = cases.device_model(gpu_pkg, synth, cfg, tensors)
    plain = cases.device_model(gpu_pkg, synth, cfg, tensors, attn_impl=1)
    tiled = cases.device_model(gpu_pkg, synth, cfg, tensors, attn_impl=2)
    M = model_io.oracle_model(cfg, tensors)
    rng = np.random.default_rng(11)
    for T in (1, 5, 63, 64, 65, 128, 129, 200, 257, 400, 750):
        x = rng.standard_normal((T, cfg.d_model)).astype(np.float32)
        a = tc.encoder_layer(0, x)
        assert np.all(np.isfinite(a))
        assert rel(a, plain.encoder_layer(0, x)) < 1e-4, T
        assert rel(a, tiled.encoder_layer(0, x)) < 1e-4, T
        if T in (65, 257):
            want = O.encoder_layer(M["layers"][0], x, O.pos_emb(T, cfg.d_model), cfg.n_heads, cfg.causal, -1, -1)
            assert rel(a, want) < 2e-4, T
    # packed batch: each item's bits equal the item alone (row stability through the new kernel)
    feats = [rng.standard_normal((n, cfg.n_mels)).astype(np.float32) for n in (1100, 40, 2500)]
    outs = tc.encoder_forward_batch(feats)
    for f, o in zip(feats, outs):
        assert np.array_equal(o, tc.encoder_forward(f))
        assert rel(o, plain.encoder_forward(f)) < 1e-4
    for m in (tc, plain, tiled):
        m.close()
