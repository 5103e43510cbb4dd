"""Glue between a synthetic tensor dictionary and the two CPU checkers —
TEST INFRASTRUCTURE ONLY.

* effective_f32(): what the reference holds after its eager GGUF block decode
  (src/weights.c:90-115): every tensor as float32.
* oracle_model(): the nested dict oracle/mynah_oracle.py works on.
* write_reference_files(): model.safetensors (+ mel_filters.safetensors) the
  compiled reference opens through its own loader.
"""
from __future__ import annotations

import os

import numpy as np

from . import mynah_oracle as O


NATIVE_Q8 = -8      # synth.NATIVE_Q8: reference-native per-row int8 with `name.scales`


def effective_f32(tensors) -> dict:
    out = {}
    for name, t in tensors.items():
        if t.ggml_type == NATIVE_Q8:
            q = t.raw.view(np.int8).reshape(t.shape)
            s = tensors[name + ".scales"].raw.view(np.float32)
            out[name] = O.dequant_int8(q, s)
        else:
            a = O.ggml_dequant(t.ggml_type, t.raw)
            out[name] = a.reshape(t.shape).astype(np.float32)
    return out


def _heads(cfg, W, M) -> None:
    """Everything after the layer stack: projector, prompt MLP, CTC head, transducer decoder, AED decoder."""
    if "encoder_projector.weight" in W:
        M["encproj_w"], M["encproj_b"] = W["encoder_projector.weight"], W["encoder_projector.bias"]
    if "prompt_projector.linear_1.weight" in W:
        for i in (1, 2):
            M[f"prompt_l{i}_w"], M[f"prompt_l{i}_b"] = W[f"prompt_projector.linear_{i}.weight"], W[f"prompt_projector.linear_{i}.bias"]
    if "ctc_head.weight" in W:
        M["ctc_w"] = W["ctc_head.weight"].reshape(W["ctc_head.weight"].shape[0], -1)
        M["ctc_b"] = W["ctc_head.bias"]
    if "decoder.embedding.weight" in W:
        nl = cfg.pred_layers
        M["dec"] = {"embedding": W["decoder.embedding.weight"], "hidden": cfg.pred_hidden, "n_layers": nl,
                    "w_ih": [W[f"decoder.lstm.weight_ih_l{l}"] for l in range(nl)],
                    "w_hh": [W[f"decoder.lstm.weight_hh_l{l}"] for l in range(nl)],
                    "b_ih": [W[f"decoder.lstm.bias_ih_l{l}"] for l in range(nl)],
                    "b_hh": [W[f"decoder.lstm.bias_hh_l{l}"] for l in range(nl)],
                    "proj_w": W["decoder.decoder_projector.weight"], "proj_b": W["decoder.decoder_projector.bias"],
                    "head_w": W["joint.head.weight"], "head_b": W["joint.head.bias"],
                    "vocab": cfg.vocab, "blank": cfg.vocab - 1, "max_symbols": cfg.max_symbols,
                    "durations": list(cfg.durations)}
    if "aed.embedding.weight" in W:
        A = {"emb": W["aed.embedding.weight"], "pos": W["aed.pos_enc"], "embln_w": W["aed.emb_norm.weight"],
             "embln_b": W["aed.emb_norm.bias"], "fin_w": W["aed.final_norm.weight"], "fin_b": W["aed.final_norm.bias"],
             "head_w": W["aed.head.weight"], "head_b": W["aed.head.bias"], "n_heads": cfg.aed_heads,
             "max_seq": cfg.aed_max_seq, "proj_w": W.get("enc_dec_proj.weight"), "proj_b": W.get("enc_dec_proj.bias"),
             "layers": []}
        for li in range(cfg.aed_layers):
            p = f"aed.layers.{li}."
            L = {}
            for nm in ("ln_self", "ln_cross", "ln_ffn"):
                L[nm + "_w"], L[nm + "_b"] = W[p + nm + ".weight"], W[p + nm + ".bias"]
            for pre, att in (("s", "self_attn"), ("c", "cross_attn")):
                for c in "qkvo":
                    L[pre + c + "_w"], L[pre + c + "_b"] = W[p + f"{att}.{c}_proj.weight"], W[p + f"{att}.{c}_proj.bias"]
            for i in (1, 2):
                L[f"ff{i}_w"], L[f"ff{i}_b"] = W[p + f"ffn.linear{i}.weight"], W[p + f"ffn.linear{i}.bias"]
            A["layers"].append(L)
        M["aed"] = A


def oracle_heads(cfg, tensors) -> dict:
    """Only the post-encoder weights (projector, heads, decoders) as the oracle wants them: the parity probes of a
    full-size model need these on the host, not the whole encoder."""
    W = {}
    for name, t in tensors.items():
        if not name.startswith("encoder.layers.") and not name.startswith("encoder.subsampling."):
            W[name] = O.ggml_dequant(t.ggml_type, t.raw).reshape(t.shape).astype(np.float32)
    M = {}
    _heads(cfg, W, M)
    return M


def oracle_model(cfg, tensors, a8=False) -> dict:
    """a8: the linears stored as reference-native int8 take int8 activations (the reference with its int8
    quantisation and MYNAH_ASR_QGEMM=1); otherwise they act through their decoded f32 values."""
    W = effective_f32(tensors)
    ss = "encoder.subsampling."
    if cfg.causal:
        cin, dw, pw = ss + "conv_in", [ss + f"layers.{i}.depthwise_conv" for i in range(2)], \
            [ss + f"layers.{i}.pointwise_conv" for i in range(2)]
    else:
        cin, dw, pw = ss + "layers.0", [ss + "layers.2", ss + "layers.5"], [ss + "layers.3", ss + "layers.6"]
    M = {"causal": bool(cfg.causal), "n_heads": cfg.n_heads, "xscale": 1.0,
         "ss": {"conv_in_w": W[cin + ".weight"], "conv_in_b": W[cin + ".bias"],
                "dw_w": [W[n + ".weight"] for n in dw], "dw_b": [W[n + ".bias"] for n in dw],
                "pw_w": [W[n + ".weight"] for n in pw], "pw_b": [W[n + ".bias"] for n in pw],
                "lin_w": W[ss + "linear.weight"], "lin_b": W[ss + "linear.bias"]},
         "layers": []}
    lin = {"ff1_w1": "feed_forward1.linear1", "ff1_w2": "feed_forward1.linear2",
           "ff2_w1": "feed_forward2.linear1", "ff2_w2": "feed_forward2.linear2",
           "q_w": "self_attn.q_proj", "k_w": "self_attn.k_proj", "v_w": "self_attn.v_proj",
           "o_w": "self_attn.o_proj", "pw1_w": "conv.pointwise_conv1", "pw2_w": "conv.pointwise_conv2"}
    for li in range(cfg.n_layers):
        p = f"encoder.layers.{li}."
        L = {}
        for short, nm in (("ln_ff1", "norm_feed_forward1"), ("ln_att", "norm_self_att"), ("ln_conv", "norm_conv"),
                          ("ln_ff2", "norm_feed_forward2"), ("ln_out", "norm_out")):
            L[short + "_w"], L[short + "_b"] = W[p + nm + ".weight"], W[p + nm + ".bias"]
        L["a8"] = bool(a8)
        for short, nm in lin.items():
            L[short] = W[p + nm + ".weight"].reshape(W[p + nm + ".weight"].shape[0], -1)
            t = tensors[p + nm + ".weight"]
            if t.ggml_type == NATIVE_Q8:
                L[short + "_q8"] = (t.raw.view(np.int8).reshape(t.shape), tensors[p + nm + ".weight.scales"].raw.view(np.float32))
            if p + nm + ".bias" in W:
                L[short + "_b"] = W[p + nm + ".bias"]
        L["relk_w"] = W[p + "self_attn.relative_k_proj.weight"]
        L["bias_u"], L["bias_v"] = W[p + "self_attn.bias_u"], W[p + "self_attn.bias_v"]
        L["dw_w"] = W[p + "conv.depthwise_conv.weight"]
        L["dw_b"] = W.get(p + "conv.depthwise_conv.bias")
        L["cnorm_w"], L["cnorm_b"] = W[p + "conv.norm.weight"], W[p + "conv.norm.bias"]
        if p + "conv.norm.running_mean" in W:   # BatchNorm fold (src/encoder.c:149-170)
            mu, var = W[p + "conv.norm.running_mean"], W[p + "conv.norm.running_var"]
            scale = (L["cnorm_w"].astype(np.float64) / np.sqrt(var.astype(np.float64) + 1e-5)).astype(np.float32)
            L["cnorm_scale"], L["cnorm_shift"] = scale, (L["cnorm_b"] - mu * scale).astype(np.float32)
        M["layers"].append(L)
    _heads(cfg, W, M)
    return M


def write_reference_files(dirpath: str, cfg, tensors, synth) -> tuple:
    """Writes model.safetensors (effective f32) and mel_filters.safetensors."""
    os.makedirs(dirpath, exist_ok=True)
    wpath = os.path.join(dirpath, "model.safetensors")
    mpath = os.path.join(dirpath, "mel_filters.safetensors")
    files = effective_f32(tensors)
    for name, t in tensors.items():       # pre-quantised form the reference maps without re-quantising (src/qmat.c:118-137)
        if t.ggml_type == NATIVE_Q8:
            files[name + ".q8"] = t.raw.view(np.int8).reshape(t.shape)
    synth.write_safetensors(wpath, files)
    synth.write_safetensors(mpath, {"mel_fb": synth.mel_filterbank(cfg.n_mels), "window": synth.hann_window()})
    return wpath, mpath
