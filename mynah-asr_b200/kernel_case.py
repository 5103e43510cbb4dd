"""One kernel on one synthetic case, for timing and for profiler captures.

    python mynah-asr_b200/kernel_case.py gemm  --T 16384 --n 4096 --k 1024 [--fast] [--iters 3]
    python mynah-asr_b200/kernel_case.py gemm  --T 16384 --n 4096 --k 1024 --fmt q8n --a8 [--iters 3]
    python mynah-asr_b200/kernel_case.py gemm  --T 32 --n 4096 --k 1024 --few-rows [--iters 3]
    python mynah-asr_b200/kernel_case.py qgemv --T 1 --n 65536 --k 4096 --fmt q4_0 [--iters 3]
    python mynah-asr_b200/kernel_case.py attention --T 750 --batch 16 [--heads 8] [--impl 0] [--iters 3]
    python mynah-asr_b200/kernel_case.py aed --batch 32 --T 250 [--positions 64] [--iters 3]

gemm : the tcgen05 contraction on resident fp16 planes (large T); with --fmt q8n --a8 the integer contraction
       (tcgen05 kind::i8) on reference-native int8 weights and int8 activation rows.
qgemv: the weight-streaming small-T kernel on the stored blocks; sizes above the 126 MB L2
       make the figure an HBM figure. Prints the CUDA-event time per launch, the algorithmic
       bytes / flops and the achieved rate.
aed  : the kernels of one AED decode position (few-row contractions, single-query self- and cross-attention,
       LayerNorms) on a Canary-1B-shaped decoder behind a tiny encoder: a profiler target that holds < 1 GB.
attention: the rel-pos self-attention kernel inside a one-layer encoder (d = 128 x heads) over a packed batch of
       `batch` segments of T frames; the time is that of the attention launches alone (device events around
       them), the flops are 6 T^2 d per segment: content scores, the needed half of the position band, P.V.
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def _pkg():
    spec = importlib.util.spec_from_file_location("mynah_asr_b200", os.path.join(HERE, "__init__.py"),
                                                  submodule_search_locations=[HERE])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["mynah_asr_b200"] = mod
    spec.loader.exec_module(mod)
    return mod


BPP = {"q8n": 1.0, "f32": 4.0, "q8_0": 34 / 32, "q4_0": 18 / 32, "q4_k": 144 / 256, "q6_k": 210 / 256}


def random_blocks(fmt: str, n: int, k: int, rng) -> np.ndarray:
    """Random but well-formed stored blocks (f16 scales around 0.005, random quants)."""
    ne = n * k
    if fmt == "f32":
        return (rng.standard_normal(ne, dtype=np.float32) * 0.02).view(np.uint8)
    geom = {"q8_0": (32, 34, [0]), "q4_0": (32, 18, [0]), "q4_k": (256, 144, [0, 2]), "q6_k": (256, 210, [208])}[fmt]
    nb = ne // geom[0]
    raw = rng.integers(0, 256, (nb, geom[1]), dtype=np.uint8)
    d = (rng.uniform(0.002, 0.008, nb)).astype(np.float16).view(np.uint8).reshape(nb, 2)
    for off in geom[2]:
        raw[:, off:off + 2] = d
    return raw.reshape(-1)


def attention_case(pkg, a, rng):
    import mynah_asr_b200.synth as synth
    T = a.T or 750
    d = 128 * a.heads
    cfg = synth.config("attention_case", d_model=d, n_layers=1, n_heads=a.heads, ffn_dim=256, n_mels=80, decoder="ctc",
                       vocab=33, wtype="q8_0")
    m = pkg.Model(synth.make_model(cfg, seed=1), n_mels=cfg.n_mels, mel_fb=synth.mel_filterbank(cfg.n_mels),
                  window=synth.hann_window(), causal=0, normalize=True, blank=cfg.vocab - 1, attn_impl=a.impl)
    feats = [rng.standard_normal((8 * T - 7, cfg.n_mels)).astype(np.float32) for _ in range(a.batch)]
    frames = m.encoder_forward_batch(feats)[0].shape[0]           # warm-up
    m.profile_begin()
    for _ in range(a.iters):
        m.encoder_forward_batch(feats)
    prof = m.profile_end()["attention"]
    ms = prof["ms"] / max(prof["launches"], 1)
    flops = 6.0 * frames * frames * d * a.batch
    print(json.dumps({"kernel": "attention", "impl": a.impl, "T": frames, "batch": a.batch, "heads": a.heads, "d": d,
                      "ms": ms, "flops": flops, "tflops": flops / (ms * 1e-3) / 1e12}))
    m.close()


def aed_case(pkg, a, rng):
    """The AED decoder of the Canary-1B shape (4 layers, d = 1024, 8 heads, FFN 4096, vocab 16384, Q8_0) behind a one-layer
    128-wide encoder, so that the process holds well under 1 GB on the device: `batch` utterances of T encoder frames,
    `iters` decodes of `--positions` positions each (no token is EOS: every decode runs to its cap)."""
    import time
    import mynah_asr_b200.synth as synth
    T = a.T or 250
    cfg = synth.config("aed_case", d_model=128, n_layers=1, n_heads=4, ffn_dim=256, n_mels=80, decoder="aed", vocab=16384,
                       aed_d=1024, aed_layers=4, aed_heads=8, aed_ffn=4096, aed_max_seq=1024, wtype="q8_0")
    m = pkg.Model(synth.make_model(cfg, seed=1), n_mels=cfg.n_mels, mel_fb=synth.mel_filterbank(cfg.n_mels),
                  window=synth.hann_window(), causal=0, normalize=True, blank=cfg.vocab - 1, aed_heads=cfg.aed_heads)
    encs = [rng.standard_normal((T, cfg.d_model)).astype(np.float32) for _ in range(a.batch)]
    prompts = [[3, 4, 5, 6, 7]] * a.batch
    caps = [a.positions - 5] * a.batch
    m.aed_decode_batch(encs, prompts, -1, caps)                   # warm-up
    t0 = time.perf_counter()
    for _ in range(a.iters):
        toks = m.aed_decode_batch(encs, prompts, -1, caps)
    dt = (time.perf_counter() - t0) / a.iters
    D, F, V, L = 1024, 4096, 16384, 4
    w_bytes = (L * (6 * D * D + 2 * D * F) + V * D) * 4.0          # fp16 (hi, lo) planes of the position's linears
    kv_bytes = L * a.batch * T * 2 * D * 4.0                        # cross K / V planes
    print(json.dumps({"kernel": "aed", "batch": a.batch, "T": T, "positions": a.positions, "tokens": int(sum(len(t) for t in toks)),
                      "ms_per_decode_wall": dt * 1e3, "us_per_position_wall": dt * 1e6 / a.positions,
                      "bytes_per_position": w_bytes + kv_bytes, "note": "wall clock around the whole call: projection of the encoder "
                      "output, cross K/V, all positions, token read-back"}))
    m.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["gemm", "qgemv", "attention", "aed"])
    ap.add_argument("--positions", type=int, default=64, help="aed: decode positions per call (prompt of 5 included)")
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--heads", type=int, default=8)
    ap.add_argument("--impl", type=int, default=0, help="attention: 0 default (tcgen05 where eligible), 2 warp-level tiled kernel")
    ap.add_argument("--T", type=int, default=0)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=1024)
    ap.add_argument("--fmt", default="q4_0", choices=list(BPP))
    ap.add_argument("--fast", action="store_true")
    ap.add_argument("--few-rows", action="store_true", help="gemm: the decoder-position kernel (weights on the 128-row side, K slices over a cluster)")
    ap.add_argument("--a8", action="store_true")
    ap.add_argument("--iters", type=int, default=3)
    a = ap.parse_args()
    pkg = _pkg()
    assert pkg.available(), "no sm_100 device"
    rng = np.random.default_rng(0)
    if a.kernel == "attention":
        return attention_case(pkg, a, rng)
    if a.kernel == "aed":
        return aed_case(pkg, a, rng)
    T = a.T or (16384 if a.kernel == "gemm" else 1)
    if a.fmt == "q8n":
        wq = rng.integers(-127, 128, (a.n, a.k), dtype=np.int8)
        q = pkg.QMat(pkg.MYNAH_Q8, wq, a.n, a.k, scales=rng.uniform(1e-4, 2e-4, a.n).astype(np.float32))
    fmt = {"q8n": pkg.MYNAH_Q8, "f32": pkg.F32, "q8_0": pkg.GGML_Q8_0, "q4_0": pkg.GGML_Q4_0, "q4_k": pkg.GGML_Q4_K, "q6_k": pkg.GGML_Q6_K}[a.fmt]
    if a.fmt != "q8n":
        q = pkg.QMat(fmt, random_blocks(a.fmt, a.n, a.k, rng), a.n, a.k)
    flags = (pkg.FAST if a.fast else pkg.A16) | (pkg.A8 if a.a8 else 0) | (pkg.FEW_ROWS if a.few_rows else 0)
    ms = q.time_ms(T, flags, a.iters)
    out = {"kernel": a.kernel, "T": T, "n": a.n, "k": a.k, "fmt": a.fmt, "ms": ms}
    if a.kernel == "gemm":
        assert T > 16 or a.few_rows
        out["flops"] = 2.0 * T * a.n * a.k
        out["tflops"] = out["flops"] / (ms * 1e-3) / 1e12
        if a.few_rows:          # a streaming kernel: operand planes of the weight (2 B per plane and element) + rows in and out
            out["bytes"] = a.n * a.k * (2.0 if a.fast else 4.0) * 1.0 + T * a.k * (2.0 if a.fast else 4.0) + T * a.n * 4
            out["gbs"] = out["bytes"] / (ms * 1e-3) / 1e9
    else:
        assert T <= 16
        out["bytes"] = a.n * a.k * BPP[a.fmt] + T * a.k * 4 + T * a.n * 4
        out["gbs"] = out["bytes"] / (ms * 1e-3) / 1e9
    print(json.dumps(out))


if __name__ == "__main__":
    main()
