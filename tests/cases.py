"""Small model shapes shared by the parity tests and the golden-fixture generator."""

TINY = {
    # Parakeet-style offline CTC, Q8_0, dk = 32 (plain attention kernel)
    "ctc_q8": dict(d_model=128, n_layers=2, n_heads=4, ffn_dim=256, n_mels=80, decoder="ctc", vocab=65,
                   wtype="q8_0"),
    # Parakeet-TDT-style, Q4_0, dk = 64 (tiled attention kernel), 2-layer LSTM, durations 0..4
    "tdt_q4": dict(d_model=256, n_layers=2, n_heads=4, ffn_dim=512, n_mels=128, decoder="tdt", vocab=97,
                   pred_hidden=64, pred_layers=2, durations=(0, 1, 2, 3, 4), wtype="q4_0", blank_bias=1.0),
    # Nemotron-style causal RNNT with LayerNorm conv norm, mixed Q4_K / Q6_K, dk = 128
    "rnnt_kq": dict(d_model=256, n_layers=2, n_heads=2, ffn_dim=512, n_mels=128, decoder="rnnt", vocab=65,
                    pred_hidden=64, pred_layers=1, wtype="q4_k", wtype_out="q6_k", causal=True, normalize=False,
                    blank_bias=2.0, max_symbols=3),
    # biases everywhere (use_bias checkpoints, e.g. parakeet-110m)
    "ctc_bias": dict(d_model=128, n_layers=1, n_heads=2, ffn_dim=256, n_mels=80, decoder="ctc", vocab=33,
                     wtype="q8_0", use_bias=True),
}

# Canary-style AED models (transformer decoder with cross-attention): decoder as wide as the
# encoder, and a narrower one behind enc_dec_proj
AED = {
    "aed_same": dict(d_model=128, n_layers=1, n_heads=4, ffn_dim=256, n_mels=80, decoder="aed", vocab=300,
                     aed_layers=2, aed_heads=4, aed_max_seq=64, wtype="q8_0"),
    "aed_proj": dict(d_model=128, n_layers=1, n_heads=4, ffn_dim=256, n_mels=80, decoder="aed", vocab=211,
                     aed_d=64, aed_layers=3, aed_heads=2, aed_ffn=192, aed_max_seq=48, wtype="q4_0"),
}
# Nemotron-style prompt-conditioned model: causal RNNT whose post-encoder MLP takes a one-hot prompt id
PROMPT = {"rnnt_prompt": dict(d_model=128, n_layers=1, n_heads=2, ffn_dim=256, n_mels=80, decoder="rnnt", vocab=49,
                              pred_hidden=64, pred_layers=1, wtype="q8_0", causal=True, normalize=False, blank_bias=1.5,
                              max_symbols=3, num_prompts=5, prompt_inter=192)}
PROMPT_IDS = (3, 0, 4)
STREAM_CONTEXTS = ((6, 0), (8, 1), (70, 0))      # (left, right) attention contexts of the streaming tests
AED_PROMPT = (7, 9, 200, 11)
AED_CAP = 24
SEEDS = {"aed_same": 4}       # weight seeds whose greedy streams do not fall into a one-token fixed point


def build(synth, name, seed=None):
    seed = SEEDS.get(name, 1) if seed is None else seed
    cfg = synth.config(name, **(TINY[name] if name in TINY else AED[name] if name in AED else PROMPT[name]))
    return cfg, synth.make_model(cfg, seed=seed)


def device_model(pkg, synth, cfg, tensors, **over):
    kw = dict(n_mels=cfg.n_mels, mel_fb=synth.mel_filterbank(cfg.n_mels), window=synth.hann_window(),
              causal=int(cfg.causal), normalize=cfg.normalize, left=cfg.left, right=cfg.right, blank=cfg.vocab - 1,
              max_symbols=cfg.max_symbols, durations=tuple(cfg.durations))
    kw.update(over)
    return pkg.Model(tensors, **kw)

# int8-activation mode (the reference's `--quant int8` with MYNAH_ASR_QGEMM=1): the ten linears of every layer stored
# in the reference-native per-row int8 format; widths are multiples of 128 as the tensor-core path wants
A8 = {
    "ctc_a8": dict(d_model=256, n_layers=2, n_heads=4, ffn_dim=512, n_mels=80, decoder="ctc", vocab=65, wtype="f32"),
    "tdt_a8": dict(d_model=256, n_layers=2, n_heads=2, ffn_dim=512, n_mels=128, decoder="tdt", vocab=97, pred_hidden=64,
                   pred_layers=1, durations=(0, 1, 2, 3, 4), wtype="f32", causal=True, normalize=False, blank_bias=1.0),
}
A8_SECONDS = {"ctc_a8": 2.5, "tdt_a8": 2.0}


def build_a8(synth, name, seed=1):
    cfg = synth.config(name, **A8[name])
    t = synth.make_model(cfg, seed=seed)
    return cfg, synth.to_native_int8(t, lambda ty, raw: raw.view("float32"))


def align_cases():
    """Seeded inputs of the alignment fixtures (the tests regenerate them): random logits with the label path made
    more or less attractive, repeated labels, the shortest possible T, flat scores (every path ties), an impossible T."""
    import numpy as np
    rng = np.random.default_rng(77)
    out = []
    for T, V, n, boost in ((40, 9, 6, 3.0), (25, 5, 12, 0.0), (120, 33, 30, 1.0), (9, 5, 3, 10.0), (64, 17, 1, 0.5), (300, 129, 70, 2.0)):
        toks = rng.integers(0, V - 1, n).tolist()
        if n > 3:
            toks[2] = toks[1]                                   # a repeated label: the blank between is mandatory
        sc = rng.standard_normal((T, V)).astype(np.float32)
        pos = np.sort(rng.choice(T, n, replace=False))
        for j, p in enumerate(pos):
            sc[p, toks[j]] += boost
        out.append((sc, toks, V - 1))
    toks = [1, 1, 2, 2, 3]
    out.append((rng.standard_normal((len(toks) + 2, 6)).astype(np.float32), toks, 5))      # T = the minimum (7)
    out.append((np.zeros((40, 5), np.float32), [0, 1, 0, 2], 4))                           # flat scores
    out.append((rng.standard_normal((3, 5)).astype(np.float32), [0, 0, 1], 4))              # impossible: needs 4 frames
    return out




# voice activity / segment planning fixtures: (seconds, seed) of synth.speech_like_audio and the segment limits
VAD_AUDIO = ((30.0, 1), (12.3, 2))
VAD_SEG_SECONDS = (5.0, 8.0)
