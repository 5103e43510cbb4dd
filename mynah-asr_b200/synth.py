"""Synthetic models and audio for the mynah-asr hot path.

The reference's published numbers were taken on real NeMo checkpoints and real
speech; neither is available offline, so tests and the benchmark use seeded
synthetic stand-ins with the same shapes and value distributions:

* weights: every tensor the reference loaders require, HF-verbatim names
  (src/encoder.c:62-143, src/subsampling.c:14-58, src/decoder.c:14-62,
  src/decoder_ctc.c:11-22), matrices ~ N(0, 0.02), norms gamma=1 beta=0,
  BatchNorm running_mean=0 running_var=1; the linears on the reference's
  quantisation allow-list (cli/main.c:268-282) stored as ggml blocks.
* audio: 16 kHz mono int16, Gaussian noise (sigma 3000) with a 4 Hz amplitude
  envelope 0.5*(1+sin(2*pi*4*t)), converted to float by /32768 as the
  reference CLI does (cli/main.c:248).

The block quantisers write valid ggml blocks (layouts as decoded by
third_party/ingot/src/dequant.c); they are simple absmax quantisers, not
ggml's search-based K-quant encoders — any valid block stream is a legitimate
weight file, and both sides of a parity test see the same effective weights.
"""
from __future__ import annotations

import json
import struct
from dataclasses import dataclass, field

import numpy as np

GGML_F32, GGML_Q4_0, GGML_Q8_0, GGML_Q4_K, GGML_Q6_K = 0, 2, 8, 12, 14
NATIVE_Q8 = -8        # not a ggml type: the reference's own per-row int8 (src/qmat.h:6-9), stored as int8 [n,k] + f32 scales [n]
GGML_NAMES = {"f32": GGML_F32, "q4_0": GGML_Q4_0, "q8_0": GGML_Q8_0, "q4_k": GGML_Q4_K, "q6_k": GGML_Q6_K}


# ----------------------------------------------------------------- quantisers
def quantize_q8_0(w: np.ndarray) -> np.ndarray:
    g = np.ascontiguousarray(w, np.float32).reshape(-1, 32)
    amax = np.abs(g).max(axis=1)
    d = (amax / 127.0).astype(np.float16)
    df = d.astype(np.float32)
    inv = np.where(df > 0, 1.0 / np.where(df > 0, df, 1), 0).astype(np.float32)
    q = np.clip(np.rint(g * inv[:, None]), -127, 127).astype(np.int8)
    out = np.empty((g.shape[0], 34), np.uint8)
    out[:, 0:2] = d.view(np.uint8).reshape(-1, 2)
    out[:, 2:] = q.view(np.uint8)
    return out.reshape(-1)


def quantize_q4_0(w: np.ndarray) -> np.ndarray:
    g = np.ascontiguousarray(w, np.float32).reshape(-1, 32)
    idx = np.abs(g).argmax(axis=1)
    mx = g[np.arange(g.shape[0]), idx]
    d = (mx / -8.0).astype(np.float16)
    df = d.astype(np.float32)
    inv = np.where(df != 0, 1.0 / np.where(df != 0, df, 1), 0).astype(np.float32)
    q = np.clip((g * inv[:, None] + 8.5).astype(np.int32), 0, 15).astype(np.uint8)
    out = np.empty((g.shape[0], 18), np.uint8)
    out[:, 0:2] = d.view(np.uint8).reshape(-1, 2)
    out[:, 2:] = q[:, :16] | (q[:, 16:] << 4)
    return out.reshape(-1)


def quantize_q4_k(w: np.ndarray) -> np.ndarray:
    """256-element super-blocks: per 32-sub-block affine (scale, min) with 6-bit
    codes relative to f16 d / dmin."""
    g = np.ascontiguousarray(w, np.float32).reshape(-1, 8, 32)
    nb = g.shape[0]
    mn = np.minimum(g.min(axis=2), 0.0)
    mxv = g.max(axis=2)
    sc = np.maximum(mxv - mn, 0) / 15.0
    d = (sc.max(axis=1) / 63.0).astype(np.float16)
    dmin = ((-mn).max(axis=1) / 63.0).astype(np.float16)
    df, dmf = d.astype(np.float32), dmin.astype(np.float32)
    ls = np.clip(np.rint(sc / np.where(df > 0, df, 1)[:, None]), 0, 63).astype(np.uint8)
    lm = np.clip(np.rint(-mn / np.where(dmf > 0, dmf, 1)[:, None]), 0, 63).astype(np.uint8)
    eff_d = df[:, None] * ls
    eff_m = dmf[:, None] * lm
    q = np.clip(np.rint((g + eff_m[:, :, None]) / np.where(eff_d > 0, eff_d, 1)[:, :, None]), 0, 15).astype(np.uint8)
    out = np.zeros((nb, 144), np.uint8)
    out[:, 0:2] = d.view(np.uint8).reshape(-1, 2)
    out[:, 2:4] = dmin.view(np.uint8).reshape(-1, 2)
    s = out[:, 4:16]
    s[:, 0:4] = (ls[:, 0:4] & 63) | ((ls[:, 4:8] >> 4) << 6)
    s[:, 4:8] = (lm[:, 0:4] & 63) | ((lm[:, 4:8] >> 4) << 6)
    s[:, 8:12] = (ls[:, 4:8] & 0x0F) | ((lm[:, 4:8] & 0x0F) << 4)
    qq = q.reshape(nb, 4, 2, 32)
    out[:, 16:] = (qq[:, :, 0, :] | (qq[:, :, 1, :] << 4)).reshape(nb, 128)
    return out.reshape(-1)


def quantize_q6_k(w: np.ndarray) -> np.ndarray:
    """256-element super-blocks: 16 sub-blocks of 16 with int8 scales, 6-bit
    quants stored as ql nibbles + qh bit pairs."""
    g = np.ascontiguousarray(w, np.float32).reshape(-1, 16, 16)
    nb = g.shape[0]
    amax = np.abs(g).max(axis=2)
    sub = amax / 31.0
    d = (sub.max(axis=1) / 127.0).astype(np.float16)
    df = d.astype(np.float32)
    sc = np.clip(np.rint(sub / np.where(df > 0, df, 1)[:, None]), 0, 127).astype(np.int8)
    eff = df[:, None] * sc.astype(np.float32)
    q = (np.clip(np.rint(g / np.where(eff > 0, eff, 1)[:, :, None]), -32, 31) + 32).astype(np.uint8)
    q = q.reshape(nb, 2, 4, 32)                 # half, quarter j, position i
    out = np.zeros((nb, 210), np.uint8)
    ql = out[:, 0:128].reshape(nb, 2, 64)
    qh = out[:, 128:192].reshape(nb, 2, 32)
    ql[:, :, 0:32] = (q[:, :, 0] & 0x0F) | ((q[:, :, 2] & 0x0F) << 4)
    ql[:, :, 32:64] = (q[:, :, 1] & 0x0F) | ((q[:, :, 3] & 0x0F) << 4)
    qh[:] = (q[:, :, 0] >> 4) | ((q[:, :, 1] >> 4) << 2) | ((q[:, :, 2] >> 4) << 4) | ((q[:, :, 3] >> 4) << 6)
    out[:, 192:208] = sc.view(np.uint8)
    out[:, 208:210] = d.view(np.uint8).reshape(-1, 2)
    return out.reshape(-1)


QUANTIZERS = {GGML_Q8_0: quantize_q8_0, GGML_Q4_0: quantize_q4_0, GGML_Q4_K: quantize_q4_k, GGML_Q6_K: quantize_q6_k}


# ------------------------------------------------------------- mel filterbank
def _hz_to_mel(f):
    f = np.asarray(f, np.float64)
    return np.where(f >= 1000.0, 15.0 + 27.0 * np.log(np.maximum(f, 1e-10) / 1000.0) / np.log(6.4), 3.0 * f / 200.0)


def _mel_to_hz(m):
    m = np.asarray(m, np.float64)
    return np.where(m >= 15.0, 1000.0 * np.exp(np.log(6.4) * (m - 15.0) / 27.0), 200.0 * m / 3.0)


def mel_filterbank(n_mels: int, n_fft: int = 512, sample_rate: int = 16000) -> np.ndarray:
    """Slaney-scale, slaney-normalised triangular filters [n_fft/2+1, n_mels]
    (the construction tools/convert_nemo.py:59-74 writes to mel_filters)."""
    n_freqs = n_fft // 2 + 1
    freqs = np.linspace(0.0, sample_rate // 2, n_freqs)
    pts = _mel_to_hz(np.linspace(_hz_to_mel(0.0), _hz_to_mel(sample_rate / 2), n_mels + 2))
    diff = pts[1:] - pts[:-1]
    slopes = pts[None, :] - freqs[:, None]
    fb = np.maximum(0.0, np.minimum(-slopes[:, :-2] / diff[:-1], slopes[:, 2:] / diff[1:]))
    fb *= 2.0 / (pts[2:] - pts[:-2])
    return fb.astype(np.float32)


def hann_window(win_length: int = 400) -> np.ndarray:
    return np.hanning(win_length).astype(np.float32)


# -------------------------------------------------------------------- configs
@dataclass
class ModelConfig:
    name: str = "tiny"
    d_model: int = 128
    n_layers: int = 2
    n_heads: int = 4
    ffn_dim: int = 512
    conv_k: int = 9
    n_mels: int = 80
    channels: int = 256
    causal: bool = False          # Nemotron-style causal convs + LayerNorm conv norm
    decoder: str = "ctc"          # "ctc" | "rnnt" | "tdt" | "aed"
    vocab: int = 129              # includes blank (last index for CTC; blank_id = vocab-1)
    pred_hidden: int = 640
    pred_layers: int = 1
    durations: tuple = ()
    max_symbols: int = 10
    wtype: str = "q8_0"           # ggml type of the allow-listed linears
    wtype_out: str = ""           # optional second type for the output projections (mixed K-quant)
    use_bias: bool = False
    blank_bias: float = 0.0       # added to the blank logit so greedy streams mix blanks and tokens
    normalize: bool = True        # per_feature mel normalisation (Parakeet); NA for Nemotron
    left: int = -1
    right: int = -1
    # AED (Canary-style transformer decoder, src/decoder_aed.h)
    aed_d: int = 0                # decoder width; != d_model adds enc_dec_proj
    aed_layers: int = 4
    aed_heads: int = 8
    aed_ffn: int = 0
    aed_max_seq: int = 1024
    aed_max_gen_delta: int = 50
    # Nemotron-style prompt-conditioned post-encoder MLP (src/encoder.c:591-614); 0 = none
    num_prompts: int = 0
    prompt_inter: int = 0
    d_out: int = field(init=False, default=0)

    def __post_init__(self):
        self.d_out = self.d_model if self.decoder in ("ctc", "aed") else self.pred_hidden
        if self.decoder == "aed":
            self.aed_d = self.aed_d or self.d_model
            self.aed_ffn = self.aed_ffn or 4 * self.aed_d


CONFIGS = {
    # Parakeet-TDT_CTC-110M-shaped, CTC head, Q8_0
    "cfg0": dict(name="cfg0", d_model=512, n_layers=17, n_heads=8, ffn_dim=2048, n_mels=80,
                 decoder="ctc", vocab=1025, wtype="q8_0"),
    # Parakeet-TDT-0.6B-shaped, Q4_0
    "cfg1": dict(name="cfg1", d_model=1024, n_layers=24, n_heads=8, ffn_dim=4096, n_mels=128,
                 decoder="tdt", vocab=8193, pred_hidden=640, pred_layers=2,
                 durations=(0, 1, 2, 3, 4), wtype="q4_0"),
    # Parakeet-RNNT-1.1B-shaped, Q4_K + Q6_K
    "cfg2": dict(name="cfg2", d_model=1024, n_layers=42, n_heads=8, ffn_dim=4096, n_mels=128,
                 decoder="rnnt", vocab=1025, pred_hidden=640, pred_layers=1, wtype="q4_k",
                 wtype_out="q6_k"),
    # Nemotron-streaming-0.6B-shaped, Q8_0
    "cfg3": dict(name="cfg3", d_model=1024, n_layers=24, n_heads=8, ffn_dim=4096, n_mels=128,
                 causal=True, decoder="rnnt", vocab=1025, pred_hidden=640, pred_layers=1,
                 wtype="q8_0", normalize=False, left=70, right=0),
    # Canary-1B-shaped AED, Q8_0
    "cfg4": dict(name="cfg4", d_model=1024, n_layers=32, n_heads=8, ffn_dim=4096, n_mels=128,
                 decoder="aed", vocab=16384, aed_layers=4, aed_heads=8, aed_ffn=4096, wtype="q8_0"),
}


def config(name: str, **over) -> ModelConfig:
    kw = dict(CONFIGS[name]) if name in CONFIGS else dict(name=name)
    kw.update(over)
    return ModelConfig(**kw)


# --------------------------------------------------------------------- models
class Tensor:
    """One named tensor: ggml type, logical shape, raw bytes."""
    __slots__ = ("name", "ggml_type", "shape", "raw")

    def __init__(self, name, ggml_type, shape, raw):
        self.name, self.ggml_type, self.shape = name, int(ggml_type), tuple(int(s) for s in shape)
        self.raw = np.ascontiguousarray(raw).view(np.uint8).reshape(-1)


def _freq_dims(n_mels: int, causal: bool):
    f = n_mels
    for _ in range(3):
        f = (f + (3 if causal else 2) - 3) // 2 + 1
    return f


def make_model(cfg: ModelConfig, seed: int = 0, weight_std: float = 0.02):
    """Returns an ordered dict name -> Tensor with every tensor the loaders need."""
    rng = np.random.default_rng(seed)
    T = {}

    def f32t(name, arr):
        T[name] = Tensor(name, GGML_F32, arr.shape, np.asarray(arr, np.float32))

    def normal(*shape):
        return rng.standard_normal(shape, dtype=np.float32) * np.float32(weight_std)

    def qlin(name, n, k, out_proj=False):
        w = normal(n, k)
        tname = cfg.wtype_out if (out_proj and cfg.wtype_out) else cfg.wtype
        gt = GGML_NAMES[tname]
        if gt in (GGML_Q4_K, GGML_Q6_K) and k % 256 != 0:
            gt = GGML_Q8_0                      # K-quant fallback, as tools/export_gguf.py:106-107
        if gt == GGML_F32:
            f32t(name, w)
        else:
            T[name] = Tensor(name, gt, (n, k), QUANTIZERS[gt](w))

    d, F, C, k = cfg.d_model, cfg.ffn_dim, cfg.channels, cfg.conv_k
    ss = "encoder.subsampling."
    if cfg.causal:
        names = dict(cin=ss + "conv_in", dw=[ss + "layers.0.depthwise_conv", ss + "layers.1.depthwise_conv"],
                     pw=[ss + "layers.0.pointwise_conv", ss + "layers.1.pointwise_conv"])
    else:
        names = dict(cin=ss + "layers.0", dw=[ss + "layers.2", ss + "layers.5"], pw=[ss + "layers.3", ss + "layers.6"])
    # fan-in-scaled conv weights keep the subsampling output O(1) (the reference
    # recipe's 0.02 would vanish through three stages; shapes are what matter)
    f32t(names["cin"] + ".weight", rng.standard_normal((C, 1, 3, 3), dtype=np.float32) / 3.0)
    f32t(names["cin"] + ".bias", np.zeros(C))
    for i in range(2):
        f32t(names["dw"][i] + ".weight", rng.standard_normal((C, 1, 3, 3), dtype=np.float32) / 3.0)
        f32t(names["dw"][i] + ".bias", np.zeros(C))
        f32t(names["pw"][i] + ".weight", rng.standard_normal((C, C, 1, 1), dtype=np.float32) / np.sqrt(C))
        f32t(names["pw"][i] + ".bias", np.zeros(C))
    CF = C * _freq_dims(cfg.n_mels, cfg.causal)
    f32t(ss + "linear.weight", rng.standard_normal((d, CF), dtype=np.float32) / np.sqrt(CF))
    f32t(ss + "linear.bias", np.zeros(d))

    for li in range(cfg.n_layers):
        p = f"encoder.layers.{li}."
        for nm in ("norm_feed_forward1", "norm_self_att", "norm_conv", "norm_feed_forward2", "norm_out"):
            f32t(p + nm + ".weight", np.ones(d)); f32t(p + nm + ".bias", np.zeros(d))
        qlin(p + "feed_forward1.linear1.weight", F, d)
        qlin(p + "feed_forward1.linear2.weight", d, F, True)
        qlin(p + "feed_forward2.linear1.weight", F, d)
        qlin(p + "feed_forward2.linear2.weight", d, F, True)
        for nm in ("q_proj", "k_proj", "v_proj"):
            qlin(p + f"self_attn.{nm}.weight", d, d)
        qlin(p + "self_attn.o_proj.weight", d, d, True)
        f32t(p + "self_attn.relative_k_proj.weight", normal(d, d))
        f32t(p + "self_attn.bias_u", normal(cfg.n_heads, d // cfg.n_heads))
        f32t(p + "self_attn.bias_v", normal(cfg.n_heads, d // cfg.n_heads))
        qlin(p + "conv.pointwise_conv1.weight", 2 * d, d)
        f32t(p + "conv.depthwise_conv.weight", rng.standard_normal((d, 1, k), dtype=np.float32) / np.sqrt(k))
        qlin(p + "conv.pointwise_conv2.weight", d, d, True)
        f32t(p + "conv.norm.weight", np.ones(d)); f32t(p + "conv.norm.bias", np.zeros(d))
        if not cfg.causal:                      # Parakeet: BatchNorm with running stats
            f32t(p + "conv.norm.running_mean", np.zeros(d)); f32t(p + "conv.norm.running_var", np.ones(d))
        if cfg.use_bias:
            for nm, n in (("feed_forward1.linear1", F), ("feed_forward1.linear2", d), ("feed_forward2.linear1", F),
                          ("feed_forward2.linear2", d), ("self_attn.q_proj", d), ("self_attn.k_proj", d),
                          ("self_attn.v_proj", d), ("self_attn.o_proj", d), ("conv.pointwise_conv1", 2 * d),
                          ("conv.depthwise_conv", d), ("conv.pointwise_conv2", d)):
                f32t(p + nm + ".bias", normal(n))

    if cfg.decoder == "ctc":
        f32t("ctc_head.weight", normal(cfg.vocab, d, 1)); f32t("ctc_head.bias", np.zeros(cfg.vocab))
    elif cfg.decoder == "aed":
        # tensor names as mynah_asr_aed_init resolves them (src/decoder_aed.c:50-113)
        D, V, FA = cfg.aed_d, cfg.vocab, cfg.aed_ffn
        f32t("aed.embedding.weight", rng.standard_normal((V, D), dtype=np.float32))
        pos = np.arange(cfg.aed_max_seq, dtype=np.float64)[:, None] / (10000.0 ** (2 * (np.arange(D) // 2) / D))[None, :]
        pe = np.where(np.arange(D)[None, :] % 2 == 0, np.sin(pos), np.cos(pos)) / np.sqrt(D)
        f32t("aed.pos_enc", pe.astype(np.float32))
        for nm in ("aed.emb_norm", "aed.final_norm"):
            f32t(nm + ".weight", 1.0 + 0.1 * rng.standard_normal(D, dtype=np.float32)); f32t(nm + ".bias", normal(D))
        qlin("aed.head.weight", V, D)
        f32t("aed.head.bias", normal(V))
        if D != d:
            qlin("enc_dec_proj.weight", D, d)
            f32t("enc_dec_proj.bias", normal(D))
        for li in range(cfg.aed_layers):
            p = f"aed.layers.{li}."
            for nm in ("ln_self", "ln_cross", "ln_ffn"):
                f32t(p + nm + ".weight", 1.0 + 0.1 * rng.standard_normal(D, dtype=np.float32)); f32t(p + nm + ".bias", normal(D))
            for att in ("self_attn", "cross_attn"):
                for nm in ("q_proj", "k_proj", "v_proj", "o_proj"):
                    # attention logits of a random model are tiny; a larger scale makes the softmax selective
                    w = rng.standard_normal((D, D), dtype=np.float32) * np.float32(4.0 / np.sqrt(D) if nm in ("q_proj", "k_proj") else 1.0 / np.sqrt(D))
                    gt = GGML_NAMES[cfg.wtype]
                    T[p + f"{att}.{nm}.weight"] = Tensor(p + f"{att}.{nm}.weight", gt, (D, D), QUANTIZERS[gt](w)) if gt != GGML_F32 \
                        else Tensor(p + f"{att}.{nm}.weight", GGML_F32, (D, D), w)
                    f32t(p + f"{att}.{nm}.bias", normal(D))
            qlin(p + "ffn.linear1.weight", FA, D); f32t(p + "ffn.linear1.bias", normal(FA))
            qlin(p + "ffn.linear2.weight", D, FA, True); f32t(p + "ffn.linear2.bias", normal(D))
    else:
        H, V, ND = cfg.pred_hidden, cfg.vocab, len(cfg.durations)
        f32t("encoder_projector.weight", rng.standard_normal((H, d), dtype=np.float32) / np.sqrt(d))
        f32t("encoder_projector.bias", np.zeros(H))
        if cfg.num_prompts:
            di = cfg.prompt_inter or 2 * d
            f32t("prompt_projector.linear_1.weight", rng.standard_normal((di, d + cfg.num_prompts), dtype=np.float32) / np.sqrt(d))
            f32t("prompt_projector.linear_1.bias", normal(di))
            f32t("prompt_projector.linear_2.weight", rng.standard_normal((d, di), dtype=np.float32) / np.sqrt(di))
            f32t("prompt_projector.linear_2.bias", normal(d))
        f32t("decoder.embedding.weight", rng.standard_normal((V, H), dtype=np.float32))
        for l in range(cfg.pred_layers):
            f32t(f"decoder.lstm.weight_ih_l{l}", rng.standard_normal((4 * H, H), dtype=np.float32) / np.sqrt(H))
            f32t(f"decoder.lstm.weight_hh_l{l}", rng.standard_normal((4 * H, H), dtype=np.float32) / np.sqrt(H))
            f32t(f"decoder.lstm.bias_ih_l{l}", np.zeros(4 * H)); f32t(f"decoder.lstm.bias_hh_l{l}", np.zeros(4 * H))
        f32t("decoder.decoder_projector.weight", rng.standard_normal((H, H), dtype=np.float32) / np.sqrt(H))
        f32t("decoder.decoder_projector.bias", np.zeros(H))
        # the joint head is on the allow-list; its scale is fan-in based so the
        # greedy stream is not a single repeated argmax
        w = rng.standard_normal((V + ND, H), dtype=np.float32) / np.sqrt(H)
        gt = GGML_NAMES[cfg.wtype]
        if gt in (GGML_Q4_K, GGML_Q6_K) and H % 256 != 0:
            gt = GGML_Q8_0
        T["joint.head.weight"] = Tensor("joint.head.weight", gt, (V + ND, H), QUANTIZERS[gt](w)) if gt != GGML_F32 \
            else Tensor("joint.head.weight", GGML_F32, (V + ND, H), w.astype(np.float32))
        hb = np.zeros(V + ND, np.float32)
        hb[V - 1] = cfg.blank_bias
        f32t("joint.head.bias", hb)
    return T


VAD_GEOMETRY = dict(frame_samples=512, context_samples=64, reflect_pad=64, n_fft=256, hop_length=128, n_bins=129,
                    stft_frames=4, encoder_channels=[128, 64, 64, 128], encoder_kernels=[3, 3, 3, 3],
                    encoder_strides=[1, 2, 2, 1], encoder_pads=[[1, 1], [1, 1], [1, 1], [1, 1]], lstm_hidden=128,
                    threshold=0.5, neg_threshold=0.35, min_speech_ms=250, min_silence_ms=100, speech_pad_ms=30)


def make_vad(seed: int = 3, head_bias: float = -2.4):
    """A voice-activity model with the geometry of Silero VAD v5 as the reference converts it
    (tools/convert_silero.py:143-215): STFT basis [2 * 129, 1, 256] (real rows, then imaginary rows, Hann-windowed
    DFT), four conv1d + ReLU blocks, one 128-wide LSTM, a 1x1 head. The network weights are random (seeded), with an
    LSTM input gain and a head scale under which the probability follows the signal's level; with the default seed
    and head bias it crosses both thresholds between the loud and the quiet stretches of speech_like_audio(). Returns (config dict for mynah.json, {name: float32 array})."""
    rng = np.random.default_rng(seed)
    g = VAD_GEOMETRY
    n_fft, nb, H = g["n_fft"], g["n_bins"], g["lstm_hidden"]
    k = np.arange(n_fft)
    win = 0.5 - 0.5 * np.cos(2.0 * np.pi * k / n_fft)
    ang = 2.0 * np.pi * np.outer(np.arange(nb), k) / n_fft
    basis = np.concatenate([np.cos(ang) * win, -np.sin(ang) * win]).astype(np.float32)[:, None, :]
    T = {"stft.forward_basis_buffer": basis}
    cin = nb
    for i, (cout, kk) in enumerate(zip(g["encoder_channels"], g["encoder_kernels"])):
        T[f"encoder.{i}.reparam_conv.weight"] = (rng.standard_normal((cout, cin, kk)) * (1.6 / np.sqrt(cin * kk))).astype(np.float32)
        T[f"encoder.{i}.reparam_conv.bias"] = (rng.standard_normal(cout) * 0.05).astype(np.float32)
        cin = cout
    T["decoder.rnn.weight_ih"] = (rng.standard_normal((4 * H, H)) * (2.0 / np.sqrt(H))).astype(np.float32)
    T["decoder.rnn.weight_hh"] = (rng.standard_normal((4 * H, H)) * (1.0 / np.sqrt(H))).astype(np.float32)
    T["decoder.rnn.bias_ih"] = (rng.standard_normal(4 * H) * 0.1).astype(np.float32)
    T["decoder.rnn.bias_hh"] = (rng.standard_normal(4 * H) * 0.1).astype(np.float32)
    T["decoder.decoder.2.weight"] = (rng.standard_normal((1, H, 1)) * 0.9).astype(np.float32)
    T["decoder.decoder.2.bias"] = np.array([head_bias], np.float32)
    cfg = {"mynah_asr_format": 1, "name": "synthetic-vad", "arch": "silero_vad_v5", "engine": "vad",
           "weights": "model.safetensors", "sample_rate": 16000, "vad": dict(g)}
    return cfg, T


def write_vad_dir(dirpath: str, cfg: dict, tensors: dict) -> None:
    import os
    os.makedirs(dirpath, exist_ok=True)
    write_safetensors(os.path.join(dirpath, "model.safetensors"), tensors)
    with open(os.path.join(dirpath, "mynah.json"), "w") as f:
        json.dump(cfg, f, indent=1)


def speech_like_audio(seconds: float, seed: int = 0, sample_rate: int = 16000) -> np.ndarray:
    """Bursts of noise of varying level separated by near-silence (0.3 - 2 s each), int16-quantised: a signal on
    which a level-sensitive detector opens and closes spans."""
    n = int(round(seconds * sample_rate))
    rng = np.random.default_rng(7000003 * (seed + 1))
    env = np.zeros(n)
    pos, loud = 0, False
    while pos < n:
        ln = int(rng.uniform(0.3, 2.0) * sample_rate)
        env[pos:pos + ln] = rng.uniform(0.3, 1.0) if loud else rng.uniform(0.0, 0.01)
        pos += ln
        loud = not loud
    x = np.clip(np.rint(6000.0 * rng.standard_normal(n) * env), -32768, 32767).astype(np.int16)
    return (x.astype(np.float32) / np.float32(32768.0)).astype(np.float32)


def quantize_rows_int8(w: np.ndarray):
    """Per-row symmetric int8 as the reference's load-time quantiser writes it (mynah_asr_quantize_int8,
    src/qmat.c:19-36): scale = amax / 127 (1 for an all-zero row), q = round-half-away(w * (1 / scale))."""
    w = np.ascontiguousarray(w, np.float32)
    amax = np.abs(w).max(axis=1)
    scale = np.where(amax > 0, amax / np.float32(127.0), np.float32(1.0)).astype(np.float32)
    v = (w * (np.float32(1.0) / scale)[:, None]).astype(np.float32)
    q = np.where(v >= 0, v + np.float32(0.5), v - np.float32(0.5)).astype(np.float32).astype(np.int32).astype(np.int8)
    return q, scale


ENCODER_LINEARS = ("feed_forward1.linear1", "feed_forward1.linear2", "feed_forward2.linear1", "feed_forward2.linear2",
                   "self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj",
                   "conv.pointwise_conv1", "conv.pointwise_conv2")


def to_native_int8(tensors: dict, decode) -> dict:
    """The same model with the ten linears of every encoder layer re-quantised to the reference-native per-row int8
    format (what `--quant int8` does to them at load, src/encoder.c:121-137): tensor `name` becomes type NATIVE_Q8
    with int8 data and `name.scales` holds the f32 row scales. decode(ggml_type, raw) -> f32 array decodes a stored
    tensor. Everything else is kept."""
    out = {}
    for name, t in tensors.items():
        if name.startswith("encoder.layers.") and name.endswith(".weight") and name.split(".", 3)[3][:-7] in ENCODER_LINEARS:
            n = t.shape[0]
            w = np.asarray(decode(t.ggml_type, t.raw), np.float32).reshape(n, -1)
            q, s = quantize_rows_int8(w)
            out[name] = Tensor(name, NATIVE_Q8, (n, w.shape[1]), q)
            out[name + ".scales"] = Tensor(name + ".scales", GGML_F32, (n,), s)
        else:
            out[name] = t
    return out


def synth_audio(seconds: float, seed: int = 0, sample_rate: int = 16000) -> np.ndarray:
    """int16-quantised Gaussian noise with a 4 Hz envelope, as float32 in [-1,1]."""
    n = int(round(seconds * sample_rate))
    rng = np.random.default_rng(1000003 * (seed + 1))
    t = np.arange(n, dtype=np.float64) / sample_rate
    env = 0.5 * (1.0 + np.sin(2.0 * np.pi * 4.0 * t))
    x = np.clip(np.rint(3000.0 * rng.standard_normal(n) * env), -32768, 32767).astype(np.int16)
    return (x.astype(np.float32) / np.float32(32768.0)).astype(np.float32)


def write_gguf(path: str, tensors: dict, alignment: int = 32) -> None:
    """name -> Tensor (ggml types only) as a GGUF v3 file: magic, version, tensor and key/value counts, the
    key/value pairs (general.architecture, general.alignment), the tensor infos (name, dims with the fastest
    dimension first, ggml type, offset into the data section), then the aligned data."""
    def s(x: str) -> bytes:
        b = x.encode()
        return struct.pack("<Q", len(b)) + b
    kv = [s("general.architecture") + struct.pack("<I", 8) + s("mynah-asr"),
          s("general.alignment") + struct.pack("<II", 4, alignment)]
    infos, blobs, off = [], [], 0
    for name, t in tensors.items():
        if t.ggml_type < 0:
            raise ValueError(f"{name}: not a ggml type")
        infos.append(s(name) + struct.pack("<I", len(t.shape)) + b"".join(struct.pack("<Q", d) for d in reversed(t.shape)) +
                     struct.pack("<IQ", t.ggml_type, off))
        blobs.append((off, t.raw))
        off += (t.raw.size + alignment - 1) // alignment * alignment
    head = b"GGUF" + struct.pack("<IQQ", 3, len(infos), len(kv)) + b"".join(kv) + b"".join(infos)
    pad = (-len(head)) % alignment
    with open(path, "wb") as f:
        f.write(head + b"\0" * pad)
        for o, raw in blobs:
            f.write(raw.tobytes())
            f.write(b"\0" * ((-raw.size) % alignment))


def write_model_file(path: str, tensors: dict) -> None:
    """A tensor dict as the reference would find it on disk: .gguf (all ggml types) or .safetensors (f32 tensors as
    they are, reference-native int8 as `<name>.q8` + `<name>.scales`)."""
    if path.endswith(".gguf"):
        write_gguf(path, tensors)
        return
    files = {}
    for name, t in tensors.items():
        if t.ggml_type == NATIVE_Q8:
            files[name + ".q8"] = t.raw.view(np.int8).reshape(t.shape)
        elif t.ggml_type == GGML_F32:
            files[name] = t.raw.view(np.float32).reshape(t.shape)
        else:
            raise ValueError(f"{name}: block-quantised tensors need a .gguf file")
    write_safetensors(path, files)


def write_safetensors(path: str, tensors: dict) -> None:
    """name -> float32 (or int8) ndarray, in the safetensors container the reference's
    loader opens (8-byte little-endian header length, JSON header, raw data)."""
    hdr, off, arrs = {}, 0, []
    for name, a in tensors.items():
        a = np.ascontiguousarray(a) if getattr(a, "dtype", None) == np.int8 else np.ascontiguousarray(a, np.float32)
        hdr[name] = {"dtype": "I8" if a.dtype == np.int8 else "F32", "shape": list(a.shape), "data_offsets": [off, off + a.nbytes]}
        off += a.nbytes
        arrs.append(a)
    js = json.dumps(hdr, separators=(",", ":")).encode()
    js += b" " * ((8 - len(js) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(js)))
        f.write(js)
        for a in arrs:
            f.write(a.tobytes())
