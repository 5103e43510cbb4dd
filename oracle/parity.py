"""Parity probes of a device model against the compiled reference — TEST INFRASTRUCTURE ONLY
(used by tests/ and by the CPU-baseline leg of bench.py, never by the product).

parity_report() runs one utterance through the unmodified reference (oracle/_ref) and through the
device library and returns what the bar is stated on, plus the diagnostics that say how much the
token comparison is worth:

* encoder output relative L2 (raw stack output and after encoder_post), strict and fast numerics;
* head logits on every frame from both encoder outputs (same host-side f32 head): per-frame argmax
  agreement, logit relative L2, and the reference's top-2 margin — the smallest over all frames and
  at the first frame whose argmax differs. For a transducer the probe uses the prediction-network
  state after SOS on every frame (logits_t = head(relu(enc_t + g0)) + bias, src/decoder.c:129-160);
* greedy tokens and frames of the whole device path against the reference's, with the number of
  distinct tokens; and teacher-forced both ways (device decoder on the reference's frames, the
  reference's decoder on the device's frames), which separates encoder error from decoder error.
"""
from __future__ import annotations

import numpy as np

from . import model_io
from . import mynah_oracle as O


def rel_l2(a, b) -> float:
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def _probe_logits(cfg, heads, enc_raw, enc):
    """[T, V] logits with bias from an encoder output: CTC head on the raw frames, transducer joint with the
    SOS state on the projected frames; None for an AED model (its decoder has no per-frame head)."""
    if cfg.decoder == "ctc":
        return (O.gemm_wt(enc_raw, heads["ctc_w"]) + heads["ctc_b"][None, :]).astype(np.float32)
    if cfg.decoder in ("rnnt", "tdt"):
        D = heads["dec"]
        H = D["hidden"]
        st = {"h": [np.zeros(H, np.float32) for _ in range(D["n_layers"])],
              "c": [np.zeros(H, np.float32) for _ in range(D["n_layers"])], "g": None}
        O._lstm_pred_step(D, st, D["blank"])
        joint = np.maximum(enc + st["g"][None, :], 0).astype(np.float32)
        V = D["vocab"]
        return (O.gemm_wt(joint, D["head_w"][:V]) + D["head_b"][None, :V]).astype(np.float32)
    return None


def _first_divergence(a, b):
    n = min(len(a), len(b))
    for i in range(n):
        if a[i] != b[i]:
            return i
    return None if len(a) == len(b) else n


def parity_report(dm, rm, cfg, tensors, audio, *, aed_prompt=None, aed_eos=None, fast=True, layerwise=False) -> dict:
    """dm: device Model (strict numerics on entry and on return), rm: ref_binding.RefModel of the same weights."""
    heads = model_io.oracle_heads(cfg, tensors)
    feats_r, valid = rm.log_mel(audio)
    feats_d, valid_d = dm.log_mel(audio)
    rep = {"audio_seconds": len(audio) / 16000.0, "mel_max_abs": float(np.abs(feats_d - feats_r).max()) if valid == valid_d else None}
    f = feats_r[:valid]
    left, right = cfg.left, cfg.right
    raw_r = rm.encoder_forward(f, left, right, raw=True)
    enc_r = raw_r if cfg.decoder == "ctc" else rm.encoder_forward(f, left, right)
    raw_d = dm.encoder_forward(f, left, right, raw=True)
    enc_d = raw_d if cfg.decoder == "ctc" else dm.encoder_forward(f, left, right)
    rep["frames"] = int(raw_r.shape[0])
    rep["encoder_rel_l2"] = {"strict_raw": rel_l2(raw_d, raw_r), "strict_post": rel_l2(enc_d, enc_r)}
    if fast:
        dm.set_strict(False)
        try:
            raw_f = dm.encoder_forward(f, left, right, raw=True)
            if cfg.decoder == "aed":
                tok_f = dm.transcribe_batch_aed([audio], aed_prompt, aed_eos, cfg.aed_max_gen_delta)[0]
            else:
                tok_f = dm.transcribe_batch([audio], 1 if cfg.decoder == "ctc" else 0)[0][0]
        finally:
            dm.set_strict(True)
        rep["encoder_rel_l2"]["fast_raw"] = rel_l2(raw_f, raw_r)
    if layerwise:
        # every layer from the reference's own input to it: what one layer adds, apart from what the stack amplifies
        x = rm.subsampling(f)
        pe = rm.pos_emb(x.shape[0])
        worst, errs = 0.0, []
        for li in range(rm.n_layers):
            xr = rm.encoder_layer(li, x, pe, left, right)
            errs.append(rel_l2(dm.encoder_layer(li, x, left, right), xr))
            x = xr
        rep["encoder_rel_l2"]["layerwise_max"] = float(max(errs))
        rep["encoder_rel_l2"]["layerwise_median"] = float(np.median(errs))
    # ---- per-frame head logits
    lg_r = _probe_logits(cfg, heads, raw_r, enc_r)
    if lg_r is not None:
        lg_d = _probe_logits(cfg, heads, raw_d, enc_d)
        top2 = np.partition(lg_r, -2, axis=1)[:, -2:]
        margin = (top2[:, 1] - top2[:, 0]).astype(np.float64)
        am_r, am_d = lg_r.argmax(1), lg_d.argmax(1)
        diff = np.nonzero(am_r != am_d)[0]
        rep["head_logits"] = {
            "probe": "CTC head on every frame" if cfg.decoder == "ctc" else "joint with the SOS prediction state on every frame",
            "argmax_agreement": float((am_r == am_d).mean()), "frames_differing": int(diff.size),
            "logit_rel_l2": rel_l2(lg_d, lg_r), "distinct_argmax": int(len(set(am_r.tolist()))),
            "ref_top2_margin_min": float(margin.min()), "ref_top2_margin_median": float(np.median(margin)),
            "ref_top2_margin_at_first_divergence": float(margin[diff[0]]) if diff.size else None,
            "logit_abs_err_max": float(np.abs(lg_d.astype(np.float64) - lg_r).max()),
        }
    # ---- tokens: whole device path, and teacher-forced both ways
    if cfg.decoder == "aed":
        cap = enc_r.shape[0] + cfg.aed_max_gen_delta
        tok_r = rm.aed_decode(enc_r, aed_prompt, aed_eos, cap).tolist()
        tok_d = dm.transcribe_batch_aed([audio], aed_prompt, aed_eos, cfg.aed_max_gen_delta)[0]
        fr_r = fr_d = None
        tf_dev = dm.aed_decode(enc_r, aed_prompt, aed_eos, cap).tolist()
        tf_ref = rm.aed_decode(enc_d, aed_prompt, aed_eos, cap).tolist()
    elif cfg.decoder == "ctc":
        tok_r, fr_r = rm.ctc_decode(raw_r)
        (tok_d, fr_d), = dm.transcribe_batch([audio], 1)
        tf_dev = dm.ctc_decode(raw_r)[0]
        tf_ref = rm.ctc_decode(raw_d)[0]
    else:
        tok_r, fr_r = rm.greedy_decode(enc_r, cfg.max_symbols)
        (tok_d, fr_d), = dm.transcribe_batch([audio], 0)
        tf_dev = dm.greedy_decode(enc_r)[0]
        tf_ref = rm.greedy_decode(enc_d, cfg.max_symbols)[0]
    fd = _first_divergence(tok_d, tok_r)
    rep["tokens"] = {"reference_tokens": len(tok_r), "device_tokens": len(tok_d), "distinct": len(set(tok_r)),
                     "identical": tok_d == tok_r, "frames_identical": None if fr_r is None else fr_d == fr_r,
                     "first_divergence": fd,
                     "device_decoder_on_reference_frames_identical": tf_dev == tok_r,
                     "reference_decoder_on_device_frames_identical": tf_ref == tok_d}
    if fast:
        rep["tokens"]["fast_mode_identical"] = list(tok_f) == list(tok_r)
        rep["tokens"]["fast_mode_first_divergence"] = _first_divergence(list(tok_f), list(tok_r))
    rep["_ref_tokens"], rep["_ref_frames"] = tok_r, fr_r
    return rep
