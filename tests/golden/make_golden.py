"""Generates tests/golden/*.npz by running the UNMODIFIED reference
(oracle/_ref/libmynah_ref.so, built by oracle/Makefile from the reference sources)
on seeded synthetic models and audio. Run in a container that has the reference:

    make -C oracle && python tests/golden/make_golden.py
    MYNAH_ASR_QGEMM=1 python tests/golden/make_golden.py ctc_a8 tdt_a8      (the int8-activation fixtures)

The fixtures pin both the numpy oracle (tests/test_oracle_pin.py) and the CUDA path
(tests/test_stages_gpu.py, tests/test_qmat_gpu.py, tests/test_aed_gpu.py, tests/test_stream_gpu.py) on machines where the reference itself is absent.
Inputs are regenerated from seeds by the tests; only reference OUTPUTS are stored.
"""
import os
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from conftest import load_package  # noqa: E402

load_package()
import mynah_asr_b200.synth as synth  # noqa: E402

import cases  # noqa: E402
from oracle import model_io, ref_binding as R  # noqa: E402

AUDIO_SECONDS = {"ctc_q8": 2.5, "tdt_q4": 3.0, "rnnt_kq": 2.0, "ctc_bias": 1.5}


def pipeline(name):
    cfg, tensors = cases.build(synth, name)
    d = tempfile.mkdtemp()
    wp, mp = model_io.write_reference_files(d, cfg, tensors, synth)
    rm = R.RefModel(wp, mp, n_mels=cfg.n_mels, normalize=int(cfg.normalize), blank=cfg.vocab - 1,
                    max_symbols=cfg.max_symbols, durations=tuple(cfg.durations), causal=int(cfg.causal))
    audio = synth.synth_audio(AUDIO_SECONDS[name], seed=7)
    feats, valid = rm.log_mel(audio)
    out = {"valid": np.int32(valid), "feats": feats}
    out["subsampling"] = rm.subsampling(feats[:valid])
    pe = rm.pos_emb(out["subsampling"].shape[0])
    out["layer0"] = rm.encoder_layer(0, out["subsampling"], pe)
    out["enc_raw"] = rm.encoder_forward(feats[:valid], raw=True)
    out["enc"] = rm.encoder_forward(feats[:valid])
    out["enc_lim"] = rm.encoder_forward(feats[:valid], left=8, right=1, raw=True)
    # a second, shorter utterance for the packed-batch path
    audio2 = synth.synth_audio(AUDIO_SECONDS[name] * 0.6, seed=8)
    f2, v2 = rm.log_mel(audio2)
    b = rm.encoder_forward_batch([feats[:valid], f2[:v2]])
    out["batch0"], out["batch1"] = b[0], b[1]
    if cfg.decoder == "ctc":
        t, f = rm.ctc_decode(out["enc_raw"])
    else:
        t, f = rm.greedy_decode(out["enc"], cfg.max_symbols)
    out["tokens"], out["frames"] = np.array(t, np.int32), np.array(f, np.int32)
    if cfg.causal:      # cache-aware streaming (mynah_asr_enc_stream_step) fed chunk by chunk, two context shapes
        for left, right in cases.STREAM_CONTEXTS:
            out[f"stream_{left}_{right}"] = rm.stream_encode(feats[:valid], left, right)
    rm.close()
    np.savez_compressed(os.path.join(HERE, f"ref_{name}.npz"), **out)
    print(name, {k: getattr(v, "shape", v) for k, v in out.items()}, "tokens", len(t), "distinct", len(set(t)))


def aed(name):
    """mynah_asr_aed_decode on the reference's own encoder output: the whole stream with an EOS
    that never fires, and the stream cut by an EOS id taken from it."""
    cfg, tensors = cases.build(synth, name)
    d = tempfile.mkdtemp()
    wp, mp = model_io.write_reference_files(d, cfg, tensors, synth)
    rm = R.RefModel(wp, mp, n_mels=cfg.n_mels, normalize=int(cfg.normalize))
    rm.aed_open(cfg.aed_layers, cfg.aed_heads, cfg.aed_max_seq, cfg.aed_max_gen_delta)
    out = {}
    for i, secs in enumerate((2.0, 1.2)):
        feats, valid = rm.log_mel(synth.synth_audio(secs, seed=11 + i))
        enc = rm.encoder_forward(feats[:valid])
        toks = rm.aed_decode(enc, cases.AED_PROMPT, -1, cases.AED_CAP)
        eos = int(toks[7])
        out[f"enc{i}"], out[f"tokens{i}"], out[f"eos{i}"] = enc, toks, np.int32(eos)
        out[f"tokens_eos{i}"] = rm.aed_decode(enc, cases.AED_PROMPT, eos, cases.AED_CAP)
        out[f"tokens_start{i}"] = rm.aed_decode(enc, cases.AED_PROMPT[:1], -1, cases.AED_CAP)
        print(name, i, "T", enc.shape[0], "tokens", len(toks), "distinct", len(set(toks.tolist())), "cut at", len(out[f"tokens_eos{i}"]))
    rm.close()
    np.savez_compressed(os.path.join(HERE, f"ref_{name}.npz"), **out)


def prompt(name):
    """mynah_asr_encoder_post with a prompt id (src/encoder.c:591-614): single, packed batch with one id per item,
    streaming, and the greedy tokens that follow."""
    cfg, tensors = cases.build(synth, name)
    d = tempfile.mkdtemp()
    wp, mp = model_io.write_reference_files(d, cfg, tensors, synth)
    rm = R.RefModel(wp, mp, n_mels=cfg.n_mels, normalize=int(cfg.normalize), blank=cfg.vocab - 1,
                    max_symbols=cfg.max_symbols, causal=int(cfg.causal))
    audio = [synth.synth_audio(s, seed=21 + i) for i, s in enumerate((1.6, 1.0, 1.3))]
    feats = []
    for a in audio:
        f, v = rm.log_mel(a)
        feats.append(f[:v])
    out = {}
    for i, pid in enumerate(cases.PROMPT_IDS):
        out[f"enc{i}"] = rm.encoder_forward(feats[i], prompt_id=pid)
        t, f = rm.greedy_decode(out[f"enc{i}"], cfg.max_symbols)
        out[f"tokens{i}"], out[f"frames{i}"] = np.array(t, np.int32), np.array(f, np.int32)
    out["enc0_p0"] = rm.encoder_forward(feats[0])
    b = rm.encoder_forward_batch(feats, prompt_ids=cases.PROMPT_IDS)
    for i in range(3):
        out[f"batch{i}"] = b[i]
    out["stream0"] = rm.stream_encode(feats[0], 6, 0, prompt_id=cases.PROMPT_IDS[0])
    rm.close()
    np.savez_compressed(os.path.join(HERE, f"ref_{name}.npz"), **out)
    print(name, {k: v.shape for k, v in out.items()}, "distinct", [len(set(out[f"tokens{i}"].tolist())) for i in range(3)])


def a8(name):
    """The reference with its int8 quantisation of the encoder linears (pre-quantised tensors, mapped as they are) and
    its threaded int8 GEMM switched on (MYNAH_ASR_QGEMM=1: int8 activations for every row count, src/qmat.c:598-643).
    The switch is read once per process, so this runs in a process of its own: `make_golden.py ctc_a8 tdt_a8`."""
    assert os.environ.get("MYNAH_ASR_QGEMM") == "1"
    cfg, tensors = cases.build_a8(synth, name)
    d = tempfile.mkdtemp()
    wp, mp = model_io.write_reference_files(d, cfg, tensors, synth)
    rm = R.RefModel(wp, mp, quant=1 + 16, n_mels=cfg.n_mels, normalize=int(cfg.normalize), blank=cfg.vocab - 1,
                    max_symbols=cfg.max_symbols, durations=tuple(cfg.durations), causal=int(cfg.causal))
    audio = synth.synth_audio(cases.A8_SECONDS[name], seed=7)
    feats, valid = rm.log_mel(audio)
    f = feats[:valid]
    out = {"enc_raw": rm.encoder_forward(f, raw=True), "enc": rm.encoder_forward(f)}
    pe = rm.pos_emb(rm.subsampling(f).shape[0])
    out["layer0"] = rm.encoder_layer(0, rm.subsampling(f), pe)
    f2, v2 = rm.log_mel(synth.synth_audio(cases.A8_SECONDS[name] * 0.5, seed=8))
    b = rm.encoder_forward_batch([f, f2[:v2]])
    out["batch0"], out["batch1"] = b[0], b[1]
    t, fr = rm.ctc_decode(out["enc_raw"]) if cfg.decoder == "ctc" else rm.greedy_decode(out["enc"], cfg.max_symbols)
    out["tokens"], out["frames"] = np.array(t, np.int32), np.array(fr, np.int32)
    rm.close()
    # the same weights through the float-activation path, to show the two modes differ by far more than the tolerance
    rf = R.RefModel(wp, mp, quant=0, n_mels=cfg.n_mels, normalize=int(cfg.normalize), causal=int(cfg.causal))
    out["enc_raw_f32"] = rf.encoder_forward(f, raw=True)
    rf.close()
    np.savez_compressed(os.path.join(HERE, f"ref_{name}.npz"), **out)
    print(name, {k: v.shape for k, v in out.items()}, "tokens", len(t), "distinct", len(set(t)),
          "a8 vs f32 rel", float(np.linalg.norm(out["enc_raw"] - out["enc_raw_f32"]) / np.linalg.norm(out["enc_raw_f32"])))


def align():
    out = {}
    for i, (sc, toks, blank) in enumerate(cases.align_cases()):
        rc, t0, t1 = R.align_ctc(sc, toks, blank)
        out[f"rc{i}"], out[f"t0_{i}"], out[f"t1_{i}"] = np.int32(rc), np.array(t0, np.int32), np.array(t1, np.int32)
        print("align", i, sc.shape, len(toks), "rc", rc)
    np.savez_compressed(os.path.join(HERE, "ref_align.npz"), **out)


def vad():
    """mynah_asr_vad_feed / _speech_spans (src/vad.c) on the synthetic Silero-shaped model, and plan_segments
    (src/mynah_asr.c:1216-1323) with and without it."""
    cfg, T = synth.make_vad()
    d = tempfile.mkdtemp()
    synth.write_vad_dir(d, cfg, T)
    rv = R.RefVad(d)
    out = {}
    for i, (secs, seed) in enumerate(cases.VAD_AUDIO):
        a = synth.speech_like_audio(secs, seed=seed)
        out[f"probs{i}"] = np.array(rv.probs(a), np.float32)
        sp = rv.speech_spans(a)
        out[f"spans{i}"] = np.array(sp, np.int64).reshape(-1, 2)
        for seg in cases.VAD_SEG_SECONDS:
            out[f"plan_energy{i}_{seg:g}"] = np.array(R.plan_segments(a, 16000, seg), np.int64).reshape(-1, 2)
            out[f"plan_vad{i}_{seg:g}"] = np.array(R.plan_segments(a, 16000, seg, rv), np.int64).reshape(-1, 2)
        print("vad", i, len(out[f"probs{i}"]), "frames", len(sp), "spans",
              {k: len(v) for k, v in out.items() if k.startswith("plan") and k[10] == str(i) or k.startswith(f"plan_vad{i}")})
    quiet = np.zeros(16000, np.float32)
    out["spans_quiet"] = np.array(rv.speech_spans(quiet), np.int64).reshape(-1, 2)
    out["plan_quiet"] = np.array(R.plan_segments(quiet, 16000, 5.0, rv), np.int64).reshape(-1, 2)
    rv.close()
    np.savez_compressed(os.path.join(HERE, "ref_vad.npz"), **out)


def qmat():
    """mynah_asr_qmat_mul on weights quantised by the reference's own load-time
    quantiser, T = 1, 4 (int8-activation dots) and 48 (dequant + sgemm): the cases
    of the reference's tests/test_qmat.c."""
    rng = np.random.default_rng(42)
    out = {}
    for n, k in ((96, 256), (40, 1024)):
        w = rng.uniform(-1, 1, (n, k)).astype(np.float32)
        out[f"w_{n}x{k}"] = w
        for T in (1, 4, 48):
            x = rng.uniform(-1, 1, (T, k)).astype(np.float32)
            out[f"x_{n}x{k}_T{T}"] = x
            for q, qn in ((0, "f32"), (1, "q8"), (2, "q4")):
                out[f"y_{n}x{k}_T{T}_{qn}"] = R.qmat_mul(w, q, x)
    np.savez_compressed(os.path.join(HERE, "ref_qmat.npz"), **out)
    print("qmat", len(out), "arrays")


if __name__ == "__main__":
    assert R.available(), "build oracle/_ref first: make -C oracle"
    only = sys.argv[1:]
    if only:                      # regenerate only the named fixtures
        for name in only:
            if name in ("align", "vad"):
                (align if name == "align" else vad)()
                continue
            (a8 if name in cases.A8 else prompt if name in cases.PROMPT else aed if name in cases.AED else pipeline)(name)
        sys.exit(0)
    for name in cases.TINY:
        pipeline(name)
    for name in cases.AED:
        aed(name)
    for name in cases.PROMPT:
        prompt(name)
    align()
    vad()
    qmat()
