"""Benchmark of the mynah-asr hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload cfg1] [--batch 16] [--seconds 60] [--mode strict|fast]

A step is one pass of the whole path (log-mel -> subsampling -> FastConformer stack ->
greedy TDT decode) over one batch of synthetic utterances. The default workload is the
Parakeet-TDT-0.6B-shaped Q4_0 model on 16 x 60 s of synthetic audio per GPU (weak
scaling: every rank decodes its own 16 utterances against a full weight replica;
nothing crosses GPUs but the final timing reduction).

Prints ONE JSON line (rank 0): metric audio-sec/sec, `value` with inputs resident in
HBM, `e2e` through the public call with host buffers (H2D of the audio and D2H of the
token ids inside the timed region), `roofline` for the contraction kernel (tensor
pipe), `cpu_baseline` = the reference's own CPU path timed on this host.
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import os
import pickle
import statistics
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
CACHE = os.path.join(tempfile.gettempdir(), "mynah_b200_bench_cache")
METRIC, UNIT = "audio-sec/sec (1/RTF)", "audio-s/s"
GEMM_TRAFFIC_RATIO = 300.5 / 352.3   # ncu dram bytes / algorithmic bytes of one contraction launch (summary under profiles/)


def load_package():
    if "mynah_asr_b200" in sys.modules:
        return sys.modules["mynah_asr_b200"]
    pkg_dir = os.path.join(ROOT, "mynah-asr_b200")
    spec = importlib.util.spec_from_file_location("mynah_asr_b200", os.path.join(pkg_dir, "__init__.py"),
                                                  submodule_search_locations=[pkg_dir])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["mynah_asr_b200"] = mod
    spec.loader.exec_module(mod)
    return mod


def shard(n_items: int, rank: int, world: int):
    """Contiguous, balanced split of item indices over ranks (utterances are independent)."""
    base, extra = divmod(n_items, world)
    lo = rank * base + min(rank, extra)
    return list(range(lo, lo + base + (1 if rank < extra else 0)))


BLANK_BIAS = {"cfg1": 2.0, "cfg2": 2.8, "cfg3": 3.7}     # overridden by --blank-bias


def workload_config(synth, name: str):
    # blank_bias puts the greedy stream at a speech-like rate (cfg1: ~3.5 tokens per second of audio)
    return synth.config(name, blank_bias=BLANK_BIAS[name]) if name in BLANK_BIAS else synth.config(name)


def recipe_std(cfg, recipe: str) -> float:
    """Standard deviation of the quantised linears. "baseline": N(0, 0.02) as the configs word it — through 17-42
    random layers the encoder output then hardly moves over time and the greedy stream repeats one token.
    "diverse": 0.32 / sqrt(d_model) (0.01 at d = 1024), under which the time-varying part of the signal
    survives the stack and the greedy stream has tens of distinct tokens; used for the supplementary parity
    report, never for the timing."""
    return 0.02 if recipe == "baseline" else 0.32 / float(np.sqrt(cfg.d_model))


def cached_model(synth, name: str, rank: int, barrier, recipe: str = "baseline", native_int8: bool = False):
    """Synthetic weights are generated once per box (rank 0) and shared through a file. native_int8: the same
    architecture and recipe with the encoder linears drawn in f32 and quantised per row to the reference-native
    int8 format, as the reference's `--quant int8` does at load (the weights of the int8-activation mode)."""
    os.makedirs(CACHE, exist_ok=True)
    cfg = workload_config(synth, name)
    path = os.path.join(CACHE, f"{name}_seed0_bb{cfg.blank_bias:g}" + ("" if recipe == "baseline" else "_" + recipe) +
                        ("_int8" if native_int8 else "") + ".pkl")
    if rank == 0 and not os.path.exists(path):
        if native_int8:
            import dataclasses
            cfg_f = dataclasses.replace(cfg, wtype="f32", wtype_out="")
            tensors = synth.to_native_int8(synth.make_model(cfg_f, seed=0, weight_std=recipe_std(cfg, recipe)),
                                           lambda ty, raw: raw.view(np.float32))
        else:
            tensors = synth.make_model(cfg, seed=0, weight_std=recipe_std(cfg, recipe))
        with open(path + ".tmp", "wb") as f:
            pickle.dump({k: (t.ggml_type, t.shape, t.raw) for k, t in tensors.items()}, f, protocol=4)
        os.replace(path + ".tmp", path)
    barrier()
    with open(path, "rb") as f:
        raw = pickle.load(f)
    return cfg, {k: synth.Tensor(k, *v) for k, v in raw.items()}


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.path = os.path.join(tempfile.gettempdir(), f"mynah_b200_clocks_{os.getpid()}.csv")
        self.gpu = gpu_index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        self.proc.wait()
        sm, mx, reasons, power = [], [], set(), []
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in open(self.path):
            p = [x.strip() for x in line.split(",")]
            if len(p) < 8:
                continue
            try:
                sm.append(float(p[0])); mx.append(float(p[1])); power.append(float(p[2]))
            except ValueError:
                continue
            for n, v in zip(names, p[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        os.unlink(self.path)
        # under load = the upper half of the samples (idle gaps between steps read low)
        sm_sorted = sorted(sm)
        load = sm_sorted[len(sm_sorted) // 2:] if sm_sorted else []
        return {"sm_mhz": statistics.median(load) if load else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


CPU_MODES = {"f32": 0, "int8": 1, "int4": 2}     # quant argument of the reference's loaders (src/qmat.h:6-9)


def ref_paths(args, cfg, tensors, synth, recipe="baseline"):
    from oracle import model_io
    d = os.path.join(CACHE, f"{args.workload}_ref" + ("" if recipe == "baseline" else "_" + recipe))
    if not os.path.exists(os.path.join(d, "model.safetensors")):
        model_io.write_reference_files(d, cfg, tensors, synth)
    return os.path.join(d, "model.safetensors"), os.path.join(d, "mel_filters.safetensors")


def ref_open(args, cfg, tensors, synth, recipe="baseline", cpu_mode="f32"):
    """The compiled reference over the same effective weights. cpu_mode f32: its default path for a ggml-quantised
    file (blocks decoded to f32 at load, OpenBLAS sgemm); int8 / int4: its own load-time quantisation of those
    weights (`--quant`, src/qmat.c:80-143: integer dots below 17 rows, dequant + sgemm above, or the threaded
    int8 GEMM above when MYNAH_ASR_QGEMM=1 is in the environment)."""
    from oracle import ref_binding as R
    wp, mp = ref_paths(args, cfg, tensors, synth, recipe)
    rm = R.RefModel(wp, mp, quant=CPU_MODES[cpu_mode], n_mels=cfg.n_mels, normalize=int(cfg.normalize), blank=cfg.vocab - 1,
                    max_symbols=cfg.max_symbols, durations=tuple(cfg.durations), causal=int(cfg.causal))
    if cfg.decoder == "aed":
        rm.aed_open(cfg.aed_layers, cfg.aed_heads, cfg.aed_max_seq, cfg.aed_max_gen_delta, quant=CPU_MODES[cpu_mode])
    return rm


def ref_transcribe(rm, cfg, audios):
    """One wave of the reference: log-mel per item, the packed-batch encoder when there are several items
    (mynah_asr_encoder_forward_batch, src/encoder.c:948-1010), greedy decoding per item."""
    feats = []
    for a in audios:
        f, v = rm.log_mel(a)
        feats.append(f[:v])
    if cfg.decoder == "ctc":
        return [rm.ctc_decode(rm.encoder_forward(f, cfg.left, cfg.right, raw=True)) for f in feats]
    encs = rm.encoder_forward_batch(feats, cfg.left, cfg.right) if len(feats) > 1 else [rm.encoder_forward(feats[0], cfg.left, cfg.right)]
    if cfg.decoder == "aed":
        out = []
        for e in encs:
            t = rm.aed_decode(e, AED_PROMPT, AED_EOS, e.shape[0] + cfg.aed_max_gen_delta).tolist()
            out.append((t, [0] * len(t)))
        return out
    return [rm.greedy_decode(e, cfg.max_symbols) for e in encs]


def ref_stream_latencies(rm, cfg, synth, seconds, seed):
    """Per-chunk wall time of the reference's cache-aware streaming encoder step on one stream
    (mynah_asr_enc_stream_step, src/encoder.c:809-872), chunks of 8 (right + 1) mel frames."""
    from oracle import ref_binding as R
    feats, valid = rm.log_mel(synth.synth_audio(seconds, seed=seed))
    mel = feats[:valid]
    es = R.lib().ref_stream_open(rm.h, cfg.left, cfg.right, cfg.n_mels)
    buf = np.empty((cfg.right + 3, rm.d_out), np.float32)
    lat, pos, frames = [], 0, 0
    while pos < mel.shape[0]:
        need = R.lib().ref_stream_need(es)
        chunk = np.ascontiguousarray(mel[pos:pos + need], np.float32)
        t0 = time.perf_counter()
        q = R.lib().ref_stream_step(es, R._fp(chunk), chunk.shape[0], mel.shape[1], int(pos + need >= mel.shape[0]), R._fp(buf))
        lat.append((time.perf_counter() - t0) * 1e3)
        if q <= 0:
            break
        frames += q
        pos += need
    R.lib().ref_stream_close(es)
    return lat, frames


def cpu_mode_name(args):
    return args.cpu_mode + ("+qgemm" if os.environ.get("MYNAH_ASR_QGEMM") == "1" else "")


def run_reference(args, rank, world):
    """--impl reference: the reference's own CPU implementation of the path on this host's cores, on a bounded
    sample of the same workload: --cpu-batch utterances per step through its packed-batch encoder (default 1;
    the GPU step is --batch of them), --cpu-mode f32 | int8 | int4, MYNAH_ASR_QGEMM=1 in the environment for
    its threaded int8 GEMM. Streaming workloads (--streams): one stream, per-chunk latency."""
    if rank != 0:
        return
    pkg = load_package()
    import mynah_asr_b200.synth as synth
    from oracle import model_io, mynah_oracle as O, ref_binding as R
    cfg, tensors = cached_model(synth, args.workload, 0, lambda: None)
    cores = os.cpu_count() or 1
    nb = args.cpu_batch
    if nb <= 0:
        # packed batches are the reference's fastest form (about +30 % from 1 to 16 utterances of 60 s on 16 cores, at
        # ~20 audio-s/s); bound the run: (steps + warm-up) x nb x seconds of audio at that rate within ~240 s
        nb = int(240.0 * 20.0 / max((args.steps + args.warmup) * args.seconds, 1e-9))
        nb = max(1, min(nb, args.batch if not args.items else 8))
    audios = [synth.synth_audio(args.seconds, seed=100 + args.sample_index + i) for i in range(nb)]
    fb, win = synth.mel_filterbank(cfg.n_mels), synth.hann_window()
    extra = {}
    if R.available():
        kind = "reference"
        rm = ref_open(args, cfg, tensors, synth, cpu_mode=args.cpu_mode)
        if args.streams > 0:
            secs = min(args.seconds, 12.0)
            def step():
                lat, frames = ref_stream_latencies(rm, cfg, synth, secs, 100)
                extra["lat"] = sorted(lat[1:]) or lat
                return frames
        else:
            def step():
                return ref_transcribe(rm, cfg, audios)
    else:
        kind = "port"
        M = model_io.oracle_model(cfg, tensors)

        def step():
            out = []
            for audio in audios:
                feats, valid = O.log_mel(audio, fb, win, normalize_per_feature=cfg.normalize)
                if cfg.decoder == "ctc":
                    out.append(O.ctc_decode(O.encoder_forward(M, feats[:valid], cfg.left, cfg.right, raw=True), M["ctc_w"], M["ctc_b"]))
                    continue
                enc = O.encoder_forward(M, feats[:valid], cfg.left, cfg.right)
                if cfg.decoder == "aed":
                    out.append(O.aed_decode(M["aed"], enc, AED_PROMPT, AED_EOS, enc.shape[0] + cfg.aed_max_gen_delta))
                else:
                    out.append(O.greedy_decode(M["dec"], enc))
            return out
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = time.perf_counter() - t0
    if args.streams > 0 and "lat" in extra:
        secs = min(args.seconds, 12.0)
        value = secs * args.steps / dt
        sample = (f"1 stream x {secs:g} s per step through the streaming encoder step, chunk by chunk "
                  f"({0.08 * (cfg.right + 1) * 1e3:g} ms chunks; the GPU step is {args.streams} streams in lock step), encoder only")
    else:
        value = args.seconds * nb * args.steps / dt
        sample = (f"{nb} utterance(s) x {args.seconds:g} s per step" +
                  (f" (the median of the {args.items} items)" if args.items else f" (of the {args.batch} x {args.seconds:g} s batch)") +
                  (", packed-batch encoder" if nb > 1 else ""))
    conf = workload_desc(args, cfg)
    conf["reference_sample"] = sample
    conf["cpu_mode"] = cpu_mode_name(args)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32" if args.cpu_mode == "f32" else args.cpu_mode, "data": "synthetic",
        "config": conf,
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": kind, "sample": sample, "mode": cpu_mode_name(args)},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    if "lat" in extra:
        lat = extra["lat"]
        pct = lambda v, p: v[min(len(v) - 1, int(round(p * (len(v) - 1))))]
        line["chunk_latency_ms"] = {"p50": pct(lat, 0.5), "p99": pct(lat, 0.99), "max": lat[-1], "streams": 1}
    print(json.dumps(line))


AED_PROMPT, AED_EOS = (3, 4, 5, 6, 7), 2     # stand-ins for the canary2 prompt and <|endoftext|>
SHAPES = {"cfg0": "Parakeet-TDT_CTC-110M", "cfg1": "Parakeet-TDT-0.6B", "cfg2": "Parakeet-RNNT-1.1B",
          "cfg3": "Nemotron-streaming-0.6B (offline path)", "cfg4": "Canary-1B"}


def item_seconds(args, rank):
    """Lengths of the length-bucketed workload of one rank: seeded U[min, max], whole 10 ms frames, ascending."""
    rng = np.random.default_rng(4000 + rank)
    return [float(v) for v in np.sort(np.round(rng.uniform(args.min_seconds, args.max_seconds, args.items), 2))]


def workload_desc(args, cfg):
    dec = {"ctc": "CTC greedy", "tdt": "TDT greedy", "rnnt": "RNNT greedy",
           "aed": f"AED greedy ({cfg.aed_layers}-layer decoder, budget T+{cfg.aed_max_gen_delta})"}[cfg.decoder]
    return {"workload": f"{args.workload}: {SHAPES.get(args.workload, args.workload)}-shaped, {cfg.n_layers} layers d={cfg.d_model} "
                        f"ffn={cfg.ffn_dim}, {cfg.wtype.upper()} weights, {dec}, "
                        + ((f"{args.items} utterances {'in all, dispatched over the GPUs longest-first' if getattr(args, 'scaling', 'weak') == 'strong' else 'per GPU'}, "
                            f"lengths U[{args.min_seconds:g}, {args.max_seconds:g}] s sorted into batches of {args.batch}") if args.items else
                           f"{args.batch} x {args.seconds:g} s {'in all' if getattr(args, 'scaling', 'weak') == 'strong' else 'per GPU'}"),
            "batch_per_gpu": args.batch, "audio_seconds": args.seconds if not args.items else "per item, see workload",
            "numerics": getattr(args, "mode", "strict"),
            "l2": "per-step working set (activations + weights, >1 GB) exceeds the 126 MB L2"}


def cpu_baseline(args, cfg, tensors, synth, model=None):
    """The reference's CPU path on a bounded sample of the workload (one utterance, f32 path, best of 2), and —
    the reference being loaded anyway — the parity report of the device model against it on that utterance."""
    from oracle import parity, ref_binding as R
    if not R.available():
        return {"value": None, "unit": UNIT, "cores": os.cpu_count(), "kind": "reference",
                "sample": "oracle/_ref not built on this box"}, None
    rm = ref_open(args, cfg, tensors, synth)
    audio = synth.synth_audio(args.seconds, seed=100 + args.sample_index)
    times = []
    for i in range(2):           # first pass warms the page cache / BLAS threads
        t0 = time.perf_counter()
        ref_transcribe(rm, cfg, [audio])
        times.append(time.perf_counter() - t0)
    # the reference's packed batch (its fastest form on this path) on a few of the step's utterances, within ~20 s
    nbp = max(1, min(args.batch if not args.items else 4, int(20.0 / max(min(times), 1e-3))))
    packed = None
    if nbp > 1:
        auds = [synth.synth_audio(args.seconds, seed=100 + args.sample_index + i) for i in range(nbp)]
        t0 = time.perf_counter()
        ref_transcribe(rm, cfg, auds)
        packed = {"value": args.seconds * nbp / (time.perf_counter() - t0), "utterances": nbp}
    rep = None
    if model is not None:
        rep = parity.parity_report(model, rm, cfg, tensors, audio, aed_prompt=AED_PROMPT, aed_eos=AED_EOS)
    rm.close()
    single = args.seconds / min(times)
    best = max(single, packed["value"]) if packed else single
    return {"value": best, "unit": UNIT, "cores": os.cpu_count(), "kind": "reference", "mode": "f32",
            "single_utterance": single, "packed_batch": packed,
            "sample": (f"the faster of: 1 utterance x {args.seconds:g} s (best of 2), and {packed['utterances']} of them through the "
                       f"packed-batch encoder (one pass)" if packed else f"1 utterance x {args.seconds:g} s, best of 2") +
                      (f" (the median of the {args.items} items of a GPU step)" if args.items else f" (the GPU step is {args.batch} of these)")}, rep


def int8_peak_tops(torch):
    """Dense int8 tensor-core rate of this GPU as a library GEMM reaches it (torch._int_mm, 8192^3, best of 10,
    CUDA events): the denominator for the int8-activation contractions. None if the library call is unavailable."""
    try:
        a = torch.randint(-127, 127, (8192, 8192), dtype=torch.int8, device="cuda")
        b = torch.randint(-127, 127, (8192, 8192), dtype=torch.int8, device="cuda")
        best = None
        for _ in range(3):
            torch._int_mm(a, b)
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); torch._int_mm(a, b); e1.record(); e1.synchronize()
            ms = e0.elapsed_time(e1)
            best = ms if best is None or ms < best else best
        return 2.0 * 8192 ** 3 / (best * 1e-3) / 1e12
    except Exception:
        return None


def hbm_roofline(pkg, synth, cfg, peaks):
    """The bandwidth-bound half of the quantised matmul, timed live: one weight matrix larger than L2 in the
    workload's own block format, streamed once per launch by the small-T kernel (qstream_tc_kernel for Q4_0 / Q8_0 /
    Q4_K, the scalar kernel otherwise) at T = 1 and T = 8 rows. achieved = algorithmic bytes
    (n k bytes-per-parameter + 4 T k + 4 T n) / average launch time (CUDA events on the kernel's stream, 50
    launches after 2 warm-up launches)."""
    fmt_of = {"q4_0": (pkg.GGML_Q4_0, synth.GGML_Q4_0, 18 / 32), "q8_0": (pkg.GGML_Q8_0, synth.GGML_Q8_0, 34 / 32),
              "q4_k": (pkg.GGML_Q4_K, synth.GGML_Q4_K, 144 / 256)}
    if cfg.wtype not in fmt_of:
        return None
    fmt, gt, bpp = fmt_of[cfg.wtype]
    n, k = 65536, 4096                                     # 151 MB of Q4_0, 285 MB of Q8_0: larger than the 126 MB L2
    rng = np.random.default_rng(7)
    w = (rng.standard_normal((2048, k), dtype=np.float32) * np.float32(0.02))
    raw = np.tile(synth.QUANTIZERS[gt](w), n // 2048)      # the same 2048 rows repeated: the kernel reads every byte anyway
    m = pkg.QMat(fmt, raw, n, k)
    peak = peaks.get("hbm_gbs") or 6650.0
    out = {"kernel": "qstream_tc_kernel (tcgen05 kind::i8, block decode fused)", "bound": "hbm", "unit": "GB/s", "peak": peak,
           "peak_source": "measured (MEASURED_PEAKS.json hbm_gbs, a device-to-device copy)" if peaks.get("hbm_gbs") else "fallback 6.65 TB/s",
           "weight": f"[{n}, {k}] {cfg.wtype.upper()}, {n * k * bpp / 1e6:.0f} MB", "rows": {}}
    for T in (1, 8):
        ms = m.time_ms(T, pkg.A16, 50)
        algo = n * k * bpp + 4.0 * T * k + 4.0 * T * n
        out["rows"][str(T)] = {"ms": ms, "achieved": algo / (ms * 1e-3) / 1e9, "frac": algo / (ms * 1e-3) / 1e9 / peak,
                               "algorithmic_bytes": algo}
    out["achieved"], out["frac"] = out["rows"]["1"]["achieved"], out["rows"]["1"]["frac"]
    out["traffic"] = out["rows"]["1"]["algorithmic_bytes"] * 1.03
    out["traffic_source"] = "estimate: algorithmic bytes x 1.03, the dram/algorithmic ratio ncu measured on this kernel and shape"
    m.close()
    return out


def timed_steps(torch, model, bhs, dec_id, steps, warmup):
    """`steps` resident passes over the uploaded batches after `warmup`: (milliseconds, per-category profile)."""
    stream = torch.cuda.ExternalStream(model.stream())
    for _ in range(warmup):
        for bh in bhs:
            model.batch_run(bh, dec_id)
    torch.cuda.synchronize()
    model.profile_begin()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(steps):
        for bh in bhs:
            model.batch_run(bh, dec_id)
    e1.record(stream)
    e1.synchronize()
    return e0.elapsed_time(e1), model.profile_end()


def a8_section(args, pkg, synth, torch, groups, dec_id, audio_s, peaks):
    """The int8-activation mode on the same architecture: encoder linears as reference-native int8 weights,
    int8 activations, integer contractions on the tensor cores (tcgen05 kind::i8). Timed like the headline
    (inputs resident), with its own roofline entry against the measured int8 rate and its own parity report
    against the reference run with the same int8 weights and MYNAH_ASR_QGEMM=1."""
    cfg, tensors = cached_model(synth, args.workload, 0, lambda: None, native_int8=True)
    dm = pkg.Model(tensors, n_mels=cfg.n_mels, mel_fb=synth.mel_filterbank(cfg.n_mels), window=synth.hann_window(),
                   causal=int(cfg.causal), normalize=cfg.normalize, left=cfg.left, right=cfg.right, blank=cfg.vocab - 1,
                   max_symbols=cfg.max_symbols, durations=tuple(cfg.durations), strict=True, aed_heads=cfg.aed_heads, a8=True)
    bhs = [dm.batch_upload(g) for g in groups]
    if dec_id == 2:
        for bh in bhs:
            dm.batch_set_aed(bh, AED_PROMPT, AED_EOS, cfg.aed_max_gen_delta)
    steps = max(2, min(args.steps, 5))
    ms, prof = timed_steps(torch, dm, bhs, dec_id, steps, 2)
    for bh in bhs:
        dm.batch_free(bh)
    g = prof["gemm"]
    achieved = g["flops"] / (g["ms"] * 1e-3) / 1e12 if g["ms"] > 0 else None
    peak = int8_peak_tops(torch)
    src = "measured: torch._int_mm 8192^3, best of 10 (burst)"
    if not peak:
        peak, src = 4500.0, "nominal dense int8 rate (the library int8 GEMM was unavailable)"
    out = {"value": audio_s * steps / (ms * 1e-3), "unit": UNIT, "ms_per_step": ms / steps, "steps": steps,
           "weights": "encoder linears per-row int8 (reference-native), the rest f32",
           "roofline": {"kernel": "gemm_i8_kernel (tcgen05 kind::i8 contraction) + the fp16 contractions of subsampling / rel-pos / projector",
                        "bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TOP/s", "frac": achieved / peak if achieved else None,
                        "peak_source": src, "frac_of_bf16_sustained": achieved / peaks["bf16_tflops_sustained"] if achieved and peaks.get("bf16_tflops_sustained") else None,
                        "launches": g["launches"], "kernel_ms_per_step": g["ms"] / steps, "flops_per_step": g["flops"] / steps},
           "breakdown_ms_per_step": {k: v["ms"] / steps for k, v in prof.items()}}
    # the integer contraction alone on the layer's shapes at this step's row count (CUDA events around 20 launches each,
    # rows quantised beforehand): what the kernel reaches where the output is wide or narrow relative to K
    rows = int(sum(len(a_) // 160 // 8 for g_ in groups for a_ in g_))
    rng = np.random.default_rng(3)
    per_shape = {}
    for n_, k_ in ((cfg.ffn_dim, cfg.d_model), (cfg.d_model, cfg.ffn_dim), (cfg.d_model, cfg.d_model)):
        qm = pkg.QMat(pkg.MYNAH_Q8, rng.integers(-127, 128, (n_, k_), dtype=np.int8), n_, k_, scales=np.full(n_, 1e-4, np.float32))
        ms_ = qm.time_ms(rows, pkg.A8, 20)
        tops = 2.0 * rows * n_ * k_ / (ms_ * 1e-3) / 1e12
        per_shape[f"[{rows} x {n_} x {k_}]"] = {"us": ms_ * 1e3, "achieved": tops, "frac": tops / peak}
        qm.close()
    out["roofline"]["per_shape_isolated"] = per_shape
    if not args.no_cpu_baseline:
        from oracle import parity, ref_binding as R
        if R.available():
            os.environ["MYNAH_ASR_QGEMM"] = "1"       # read once, at the reference's first many-row quantised product
            wp, mp = ref_paths(args, cfg, tensors, synth, recipe="int8")
            rm = R.RefModel(wp, mp, quant=1 + 16, n_mels=cfg.n_mels, normalize=int(cfg.normalize), blank=cfg.vocab - 1,
                            max_symbols=cfg.max_symbols, durations=tuple(cfg.durations), causal=int(cfg.causal))
            if cfg.decoder == "aed":
                rm.aed_open(cfg.aed_layers, cfg.aed_heads, cfg.aed_max_seq, cfg.aed_max_gen_delta)
            audio = synth.synth_audio(args.seconds, seed=100 + args.sample_index)
            t0 = time.perf_counter()
            ref_transcribe(rm, cfg, [audio])
            ref_s = time.perf_counter() - t0
            rep = parity.parity_report(dm, rm, cfg, tensors, audio, aed_prompt=AED_PROMPT, aed_eos=AED_EOS, fast=False, layerwise=True)
            rm.close()
            rep["reference"] = "oracle/_ref with the same int8 encoder weights (mapped pre-quantised), joint head f32, MYNAH_ASR_QGEMM=1"
            out["parity"] = {k: v for k, v in rep.items() if not k.startswith("_")}
            out["cpu_baseline"] = {"value": args.seconds / ref_s, "unit": UNIT, "cores": os.cpu_count(), "kind": "reference",
                                   "mode": "int8+qgemm", "sample": f"1 utterance x {args.seconds:g} s, one pass"}
    dm.close()
    return out


def parity_diverse(args, pkg, synth, seconds):
    """Supplementary parity report on a second seeded model of the same architecture whose weights keep the
    encoder output varying over time (recipe "diverse"), so that the full-size greedy stream has many distinct
    tokens. One utterance; nothing here is timed."""
    from oracle import parity, ref_binding as R
    if not R.available():
        return None
    cfg, tensors = cached_model(synth, args.workload, 0, lambda: None, recipe="diverse")
    dm = pkg.Model(tensors, n_mels=cfg.n_mels, mel_fb=synth.mel_filterbank(cfg.n_mels), window=synth.hann_window(),
                   causal=int(cfg.causal), normalize=cfg.normalize, left=cfg.left, right=cfg.right, blank=cfg.vocab - 1,
                   max_symbols=cfg.max_symbols, durations=tuple(cfg.durations), strict=True, aed_heads=cfg.aed_heads)
    rm = ref_open(args, cfg, tensors, synth, recipe="diverse")
    audio = synth.synth_audio(seconds, seed=100 + args.sample_index)
    rep = parity.parity_report(dm, rm, cfg, tensors, audio, aed_prompt=AED_PROMPT, aed_eos=AED_EOS)
    rm.close()
    dm.close()
    rep["recipe"] = f"diverse: linears ~ N(0, 0.32 / sqrt(d_model)) = N(0, {recipe_std(cfg, 'diverse'):.4f}), seed 0"
    return {k: v for k, v in rep.items() if not k.startswith("_")}


def run_streaming(args, pkg, synth, torch, dist, cfg, tensors, model, rank, world, local, barrier):
    """--streams N: N concurrent streams per GPU through the cache-aware streaming encoder step in lock step
    (one step = one chunk of 8 (right + 1) mel frames = 80 (right + 1) ms of audio per stream). Steady state:
    the K/V caches are full before the timed region. Encoder step only; greedy decoding runs on the
    collected frames at stream end, as in the tests."""
    left, right = cfg.left, cfg.right
    q = right + 1
    chunk_mel, chunk_s = 8 * q, 0.08 * q
    # --scaling strong: --streams is the total, every stream stays on one GPU (contiguous blocks);
    # weak: --streams per GPU
    import mynah_asr_b200.dispatch as dispatch
    S = len(dispatch.sticky_streams(args.streams, world)[rank]) if args.scaling == "strong" else args.streams
    S_total = args.streams if args.scaling == "strong" else args.streams * world
    # a step feeds --chunk-ms of audio per stream: n_sub consecutive chunks of the encoder's own size
    n_sub = max(1, int(round(args.chunk_ms / (chunk_s * 1e3)))) if args.chunk_ms else 1
    step_s = chunk_s * n_sub
    grp = model.stream_open(S, left, right)
    lib = pkg.lib()
    # one long synthetic utterance supplies mel frames; stream s reads it at offset 13 s frames
    feats, valid = model.log_mel(synth.synth_audio(60.0, seed=100 + rank))
    feats = feats[:valid]
    def chunk_for(step, n):
        idx = (np.arange(S)[:, None] * 13 + step * chunk_mel + np.arange(n)[None, :]) % (valid - 1)
        return np.ascontiguousarray(feats[idx], np.float32)              # [S, n, n_mels]
    fill = (left + q - 1) // q + 2                                       # steps until every cache is full
    stream = torch.cuda.ExternalStream(model.stream())
    step_no = 0
    first = chunk_for(0, grp.need())
    grp.step(first)
    step_no += 1
    dev_in = torch.empty((S, chunk_mel, cfg.n_mels), dtype=torch.float32, device="cuda")
    dev_out = torch.empty((S, q + 2, cfg.d_out), dtype=torch.float32, device="cuda")
    pinned = torch.empty((S, chunk_mel, cfg.n_mels), dtype=torch.float32).pin_memory()
    def dev_step():
        rc = lib.mynah_b200_stream_step_device(grp.h, dev_in.data_ptr(), chunk_mel, 0, dev_out.data_ptr())
        if rc < 0:
            raise SystemExit("stream_step_device failed: " + pkg._err())
    for _ in range(fill + args.warmup):
        dev_in.copy_(torch.from_numpy(chunk_for(step_no, chunk_mel)))
        torch.cuda.synchronize()
        dev_step()
        step_no += 1
    torch.cuda.synchronize()
    clocks = ClockSampler(local)
    barrier()
    if rank == 0:
        clocks.start()
    pkg.launch_count(reset=True)
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    barrier()
    t_all0 = torch.cuda.Event(enable_timing=True); t_all1 = torch.cuda.Event(enable_timing=True)
    t_all0.record(stream)
    for a, b in evs:                                                     # value: chunks already resident in HBM
        a.record(stream)
        for _ in range(n_sub):
            dev_step()
        b.record(stream)
    t_all1.record(stream)
    t_all1.synchronize()
    barrier()
    launches = pkg.launch_count()
    ms = t_all0.elapsed_time(t_all1)
    lat = sorted(a.elapsed_time(b) for a, b in evs)
    clk = clocks.stop() if rank == 0 else None
    # per-launch spans of the contractions (the roofline figures) come from a few extra steps: with spans on,
    # the step is issued launch by launch instead of replaying its captured graph
    prof_steps = min(args.steps, 5)
    model.profile_begin()
    for _ in range(prof_steps):
        dev_step()
    torch.cuda.synchronize()
    prof = model.profile_end()
    # e2e: the public call with host buffers — mel chunk H2D, encoder step, greedy decoding of the chunk with the
    # transducer state carried on the device, new token ids D2H — all inside the timed region
    host_chunks = [chunk_for(step_no + i, chunk_mel) for i in range(args.steps * n_sub + 2)]
    e2e_lat, n_tok = [], 0
    for c in host_chunks[:2]:                                            # warm-up (first decode call builds the state)
        grp.step_decode(c)
    barrier()
    t0 = time.perf_counter()
    for i in range(args.steps):
        t1 = time.perf_counter()
        for c in host_chunks[2 + i * n_sub:2 + (i + 1) * n_sub]:
            pinned.copy_(torch.from_numpy(c))
            res = grp.step_decode(pinned.numpy())
            n_tok += sum(len(t) for t, _ in res)
        e2e_lat.append((time.perf_counter() - t1) * 1e3)
    e2e_ms = (time.perf_counter() - t0) * 1e3
    barrier()
    grp.close()
    t = torch.tensor([ms, e2e_ms], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_max, e2e_max = t.tolist()
    if rank != 0:
        return
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except OSError:
        pass
    peak_tf = peaks.get("bf16_tflops_sustained") or 1590.0
    g = prof["gemm"]
    achieved = g["flops"] / (g["ms"] * 1e-3) / 1e12 if g["ms"] > 0 else None
    pct = lambda v, p: v[min(len(v) - 1, int(round(p * (len(v) - 1))))]
    e2e_sorted = sorted(e2e_lat)
    print(json.dumps({
        "metric": METRIC, "value": S_total * step_s * args.steps / (ms_max * 1e-3), "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_max / args.steps, "higher_is_better": True,
        "scaling": args.scaling, "vs_baseline": None,
        "dtype": "f16 x3 split (f32 accumulate)" if args.mode == "strict" else "f16 (f32 accumulate)", "data": "synthetic",
        "config": {"workload": f"{args.workload}: {SHAPES.get(args.workload, args.workload)}-shaped cache-aware streaming, {cfg.n_layers} layers "
                               f"d={cfg.d_model}, {cfg.wtype.upper()} weights, left {left} right {right}, {S_total} streams over {world} GPU(s) "
                               f"({S} on rank 0, each stream stays on its GPU) in lock step, {step_s * 1e3:g} ms of audio per stream and step "
                               f"= {n_sub} chunk(s) of the encoder's {chunk_s * 1e3:g} ms, caches full; value = encoder steps, "
                               f"e2e = encoder steps + per-chunk greedy decoding",
                   "streams_total": S_total, "streams_rank0": S, "step_seconds": step_s, "chunk_seconds": chunk_s, "numerics": args.mode,
                   "l2": "weights (> 600 MB) exceed the 126 MB L2"},
        "chunk_latency_ms": {"p50": pct(lat, 0.5), "p99": pct(lat, 0.99), "max": lat[-1],
                             "e2e_p50": pct(e2e_sorted, 0.5), "e2e_p99": pct(e2e_sorted, 0.99),
                             "per": f"step of {step_s * 1e3:g} ms of audio per stream (rank 0)"},
        "e2e": {"value": S_total * step_s * args.steps / (e2e_max * 1e-3), "unit": UNIT,
                "h2d_bytes_per_step": int(S * chunk_mel * n_sub * cfg.n_mels * 4), "d2h_bytes_per_step": int(8 * n_tok / max(args.steps, 1)),
                "includes": "encoder step + per-chunk greedy decoding", "tokens_per_step": n_tok / max(args.steps, 1)},
        "gpu_launches": launches,
        "roofline": {"kernel": "gemm_tc_kernel (tcgen05 contraction)", "bound": "tensor", "achieved": achieved, "peak": peak_tf,
                     "unit": "TFLOP/s", "frac": achieved / peak_tf if achieved else None,
                     "traffic": g["bytes"] / prof_steps * GEMM_TRAFFIC_RATIO, "traffic_unit": "bytes per chunk (all contraction launches)",
                     "traffic_source": "estimate: algorithmic bytes x 0.853, the dram/algorithmic ratio ncu measured on one launch",
                     "launches": g["launches"], "kernel_ms_per_chunk": g["ms"] / prof_steps, "flops_per_chunk": g["flops"] / prof_steps,
                     "mma_flops_multiplier": 3 if args.mode == "strict" else 1},
        "clocks": clk,
        "cpu_baseline": stream_cpu_baseline(args, cfg, tensors, synth) if world == 1 and not args.no_cpu_baseline else
                        {"value": None, "unit": UNIT, "cores": os.cpu_count(), "kind": "reference", "sample": "timed at N=1 only"},
    }))


def stream_cpu_baseline(args, cfg, tensors, synth):
    """One stream through the reference's streaming encoder step on this host, chunk by chunk (bounded: 10 s)."""
    from oracle import ref_binding as R
    if not R.available():
        return {"value": None, "unit": UNIT, "cores": os.cpu_count(), "kind": "reference", "sample": "oracle/_ref not built on this box"}
    rm = ref_open(args, cfg, tensors, synth)
    secs = 10.0
    t0 = time.perf_counter()
    lat, frames = ref_stream_latencies(rm, cfg, synth, secs, 100)
    dt = time.perf_counter() - t0
    rm.close()
    lat = sorted(lat[1:]) or lat
    pct = lambda v, p: v[min(len(v) - 1, int(round(p * (len(v) - 1))))]
    return {"value": secs / dt, "unit": UNIT, "cores": os.cpu_count(), "kind": "reference", "mode": "f32",
            "sample": f"1 stream x {secs:g} s through mynah_asr_enc_stream_step chunk by chunk (encoder only; the GPU step is {args.streams} streams)",
            "chunk_latency_ms": {"p50": pct(lat, 0.5), "p99": pct(lat, 0.99), "chunk_ms": 80 * (cfg.right + 1)}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg1")
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--seconds", type=float, default=60.0)
    ap.add_argument("--items", type=int, default=None,
                    help="length-bucketed workload: utterances per GPU with lengths ~ U[--min-seconds, --max-seconds], sorted "
                         "and cut into batches of --batch (default for cfg2: 256 items in batches of 64)")
    ap.add_argument("--min-seconds", type=float, default=5.0)
    ap.add_argument("--max-seconds", type=float, default=120.0)
    ap.add_argument("--streams", type=int, default=0, help="causal workloads: concurrent streams per GPU through the streaming step")
    ap.add_argument("--mode", default="strict", choices=["strict", "fast"])
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"],
                    help="weak: the workload per GPU is fixed; strong: ONE seeded workload (all --items, or all --streams) is "
                         "dispatched over the GPUs (longest-first buckets offline, sticky streams online)")
    ap.add_argument("--chunk-ms", type=float, default=0.0, help="streaming: audio fed per stream and step (a multiple of the encoder's chunk)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--skip-e2e", action="store_true", help="profiling runs: only the resident-input timing")
    ap.add_argument("--blank-bias", type=float, default=None, help="bias of the blank logit of the synthetic transducer head")
    ap.add_argument("--cpu-mode", default="f32", choices=list(CPU_MODES), help="reference arm: f32 (blocks decoded at load + sgemm), "
                    "or the reference's own int8 / int4 load-time quantisation; MYNAH_ASR_QGEMM=1 in the environment adds its threaded int8 GEMM")
    ap.add_argument("--cpu-batch", type=int, default=0, help="reference arm: utterances per step through its packed-batch encoder "
                    "(0 = as many of the GPU step's utterances as keep the whole run within about four minutes)")
    ap.add_argument("--no-extra", action="store_true", help="skip the extra sections (fast numerics, batch 1, int8-activation mode)")
    ap.add_argument("--no-diverse", action="store_true", help="skip the supplementary parity report on the diverse-recipe model")
    args = ap.parse_args()
    defaults = {"cfg0": (1, 30.0), "cfg4": (32, 20.0)}           # batch, seconds as the configs word them
    if args.workload in defaults:
        if args.batch == 16:
            args.batch = defaults[args.workload][0]
        if args.seconds == 60.0:
            args.seconds = defaults[args.workload][1]
    if args.items is None:
        args.items = 256 if args.workload == "cfg2" else 0
        if args.items and args.batch == 16:
            args.batch = 64
    if args.items:
        args.seconds = item_seconds(args, 0)[args.items // 2]          # the reference arm's sample: the median item
    args.sample_index = args.items // 2 if args.items else 0
    if args.blank_bias is not None and args.workload in BLANK_BIAS:
        BLANK_BIAS[args.workload] = args.blank_bias
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        if args.steps == 5 and args.warmup == 3:
            args.steps, args.warmup = 2, 1
        run_reference(args, rank, world)
        return

    import torch
    import torch.distributed as dist
    pkg = load_package()
    import mynah_asr_b200.synth as synth
    torch.cuda.set_device(local)
    if pkg.lib().mynah_b200_select_device(local) < 0:
        raise SystemExit("device selection failed")
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    cfg, tensors = cached_model(synth, args.workload, rank, barrier)
    t_load = time.perf_counter()
    model = pkg.Model(tensors, n_mels=cfg.n_mels, mel_fb=synth.mel_filterbank(cfg.n_mels),
                      window=synth.hann_window(), causal=int(cfg.causal), normalize=cfg.normalize, left=cfg.left,
                      right=cfg.right, blank=cfg.vocab - 1, max_symbols=cfg.max_symbols,
                      durations=tuple(cfg.durations), strict=args.mode == "strict", aed_heads=cfg.aed_heads)
    t_load = time.perf_counter() - t_load
    load_stats = model.load_stats()
    dec_id = {"ctc": 1, "aed": 2}.get(cfg.decoder, 0)
    if args.streams > 0:
        if not cfg.causal or cfg.left < 0:
            raise SystemExit("--streams needs a causal workload with a limited context (cfg3)")
        run_streaming(args, pkg, synth, torch, dist, cfg, tensors, model, rank, world, local, barrier)
        if world > 1:
            dist.destroy_process_group()
        return
    # this rank's utterances: global item ids shard over ranks (weak scaling: batch per GPU fixed)
    import mynah_asr_b200.dispatch as dispatch
    strong = None
    if args.scaling == "strong":
        # ONE seeded workload for every N: all ranks compute the same assignment from the lengths alone
        all_secs = item_seconds(args, 0) if args.items else [args.seconds] * args.batch
        parts = dispatch.lpt_assign(all_secs, world, bucket=args.batch)
        mine = [i for b in dispatch.rank_batches(parts[rank], all_secs, args.batch) for i in b]
        secs, seeds = [all_secs[i] for i in mine], [100 + i for i in mine]
        strong = {"items_total": len(all_secs), "items_per_rank": [len(p_) for p_ in parts],
                  "imbalance_modelled": dispatch.imbalance(all_secs, parts), "mine": mine, "audio_total_s": float(sum(all_secs))}
    elif args.items:
        secs = item_seconds(args, rank)
        seeds = [100 + rank * args.items + i for i in range(args.items)]
    else:
        items = shard(args.batch * world, rank, world)
        secs, seeds = [args.seconds] * len(items), [100 + it for it in items]
    lens = [int(round(v * 16000)) for v in secs]
    pinned = torch.empty(sum(lens), dtype=torch.float32).pin_memory()
    audio, off = [], 0
    for v, sd, n in zip(secs, seeds, lens):
        pinned[off:off + n].copy_(torch.from_numpy(synth.synth_audio(v, seed=sd)[:n]))
        audio.append(pinned[off:off + n].numpy())
        off += n
    audio_s = sum(lens) / 16000.0
    # one batch per step, or the sorted items cut into batches that a step runs one after the other
    groups = [audio[i:i + args.batch] for i in range(0, len(audio), args.batch)]
    stream = torch.cuda.ExternalStream(model.stream())

    # ---- value: inputs resident in HBM
    bhs = [model.batch_upload(g) for g in groups]
    if dec_id == 2:
        for bh in bhs:
            model.batch_set_aed(bh, AED_PROMPT, AED_EOS, cfg.aed_max_gen_delta)

    def resident_step():
        for bh in bhs:
            model.batch_run(bh, dec_id)

    def public_call():
        out = []
        for g in groups:
            if dec_id == 2:
                out += [(t, [0] * len(t)) for t in model.transcribe_batch_aed(g, AED_PROMPT, AED_EOS, cfg.aed_max_gen_delta)]
            else:
                out += model.transcribe_batch(g, dec_id)
        return out

    for _ in range(args.warmup):
        resident_step()
    clocks = ClockSampler(local)
    barrier()
    if rank == 0:
        clocks.start()
    pkg.launch_count(reset=True)
    model.profile_begin()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record(stream)
    for _ in range(args.steps):
        resident_step()
    e1.record(stream)
    e1.synchronize()
    barrier()
    launches = pkg.launch_count()
    prof = model.profile_end()
    ms = e0.elapsed_time(e1)
    clk = clocks.stop() if rank == 0 else None
    resident_tokens = []
    for bh, g in zip(bhs, groups):
        resident_tokens += model.batch_fetch(bh, len(g))
        model.batch_free(bh)

    # ---- e2e: the public call with host (pinned) buffers, copies inside the timed region
    if args.skip_e2e:
        res, e2e_ms = resident_tokens, float("nan")
    else:
        for _ in range(min(args.warmup, 2)):
            public_call()
        barrier()
        t0 = time.perf_counter()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record(stream)
        for _ in range(args.steps):
            res = public_call()
        f1.record(stream)
        f1.synchronize()
        e2e_ms = max(f0.elapsed_time(f1), (time.perf_counter() - t0) * 1e3)
        barrier()
        assert [r[0] for r in res] == [r[0] for r in resident_tokens], "resident and e2e paths disagree"
    h2d = sum(a.nbytes for a in audio)
    d2h = sum(8 * len(r[0]) for r in res)

    t = torch.tensor([ms, e2e_ms], dtype=torch.float64, device="cuda")
    per_rank = [t.clone() for _ in range(world)]
    if world > 1:
        dist.all_gather(per_rank, t)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_max, e2e_max = t.tolist()
    total_audio = strong["audio_total_s"] if strong else audio_s * world
    if strong:
        # transcripts gathered on the host by item index (the only thing that crosses ranks, off the timed path)
        part = {i: r for i, r in zip(strong.pop("mine"), res)}
        parts_all = [None] * world
        if world > 1:
            dist.all_gather_object(parts_all, part)
        else:
            parts_all = [part]
        merged = dispatch.gather_by_index(parts_all, strong["items_total"])
        busy = [float(p_[0]) / args.steps for p_ in per_rank]
        strong.update({"per_rank_ms_per_step": busy, "imbalance_measured": max(busy) / (sum(busy) / len(busy)),
                       "transcripts_gathered": len(merged), "tokens_total": sum(len(r[0]) for r in merged)})

    if rank == 0:
        import json as _json
        peaks = {}
        try:
            peaks = _json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except OSError:
            pass
        peak_tf = peaks.get("bf16_tflops_sustained")
        peak_src = "measured (MEASURED_PEAKS.json bf16_tflops_sustained: kernel timed inside a long step)"
        if not peak_tf:
            peak_tf, peak_src = 1590.0, "fallback 1.59 PFLOP/s (MEASURED_PEAKS.json absent)"
        g = prof["gemm"]
        achieved = g["flops"] / (g["ms"] * 1e-3) / 1e12 if g["ms"] > 0 else None
        line = {
            "metric": METRIC, "value": total_audio * args.steps / (ms_max * 1e-3), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_max / args.steps, "higher_is_better": True,
            "scaling": args.scaling, "vs_baseline": None,
            "dtype": "f16 x3 split (f32 accumulate)" if args.mode == "strict" else "f16 (f32 accumulate)",
            "data": "synthetic", "config": workload_desc(args, cfg),
            "e2e": {"value": total_audio * args.steps / (e2e_max * 1e-3), "unit": UNIT,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": launches,
            "roofline": {"kernel": "gemm_tc_kernel (tcgen05 contraction)", "bound": "tensor",
                         "achieved": achieved, "peak": peak_tf, "unit": "TFLOP/s",
                         "frac": achieved / peak_tf if achieved else None, "peak_source": peak_src,
                         # DRAM bytes of the contraction launches of one step: their algorithmic bytes (operand
                         # planes once, output once) times the ratio an ncu capture of one launch measured
                         # ([16384 x 4096 x 1024], dram read + write = 300.5 MB for 352.3 MB algorithmic: part
                         # of the output is still in L2 when the kernel ends)
                         "traffic": g["bytes"] / args.steps * GEMM_TRAFFIC_RATIO,
                         "traffic_unit": "bytes per step (all contraction launches)",
                         "traffic_source": "estimate: algorithmic bytes x 0.853, the dram/algorithmic ratio ncu measured on one launch",
                         "algorithmic_bytes_per_step": g["bytes"] / args.steps,
                         "launches": g["launches"], "kernel_ms_per_step": g["ms"] / args.steps,
                         "flops_per_step": g["flops"] / args.steps,
                         "mma_flops_multiplier": 3 if args.mode == "strict" else 1},
            "breakdown_ms_per_step": {k: v["ms"] / args.steps for k, v in prof.items()},
            "tokens_per_step": sum(len(r[0]) for r in res),
            "decoder_clocks": dict(zip(("head_mma", "head_barrier", "select", "lstm", "proj", "steps", "emit_steps", "head_stage"),
                                       model.decoder_clocks())),
            "clocks": clk,
        }
        line["model_load"] = {"seconds_host_call": t_load, "seconds_upload_and_decode": load_stats["seconds"],
                              "host_bytes": load_stats["host_bytes"], "device_slab_bytes": load_stats["device_slab_bytes"],
                              "what": "tensors handed over by name, copied through pinned staging into device slabs, blocks re-tiled "
                                      "and decoded to operand planes by kernels (the reference decodes GGUF blocks to f32 on the host)"}
        if strong:
            line["dispatch"] = strong
        if world == 1 and not args.no_extra and args.mode == "strict":
            # fast numerics (one fp16 product per term) on the same model and inputs; its accuracy is in `parity`
            model.set_strict(False)
            bh2 = [model.batch_upload(g_) for g_ in groups]
            if dec_id == 2:
                for bh in bh2:
                    model.batch_set_aed(bh, AED_PROMPT, AED_EOS, cfg.aed_max_gen_delta)
            fsteps = max(2, min(args.steps, 5))
            fms, fprof = timed_steps(torch, model, bh2, dec_id, fsteps, 2)
            model.set_strict(True)
            fg = fprof["gemm"]
            fach = fg["flops"] / (fg["ms"] * 1e-3) / 1e12 if fg["ms"] > 0 else None
            line["fast"] = {"value": audio_s * fsteps / (fms * 1e-3), "unit": UNIT, "ms_per_step": fms / fsteps,
                            "roofline": {"kernel": "gemm_tc_kernel<.,1>", "bound": "tensor", "achieved": fach, "peak": peak_tf,
                                         "unit": "TFLOP/s", "frac": fach / peak_tf if fach else None,
                                         "kernel_ms_per_step": fg["ms"] / fsteps},
                            "note": "single fp16 product per term; encoder rel-L2 against the reference under parity.encoder_rel_l2.fast_raw"}
            if not args.items and args.batch > 1:
                # one utterance per step (the configuration is quoted at batch 1 as well)
                one = [model.batch_upload(groups[0][:1])]
                if dec_id == 2:
                    model.batch_set_aed(one[0], AED_PROMPT, AED_EOS, cfg.aed_max_gen_delta)
                bms, _ = timed_steps(torch, model, one, dec_id, 5, 2)
                model.batch_free(one[0])
                t0 = time.perf_counter()
                for _ in range(5):
                    model.transcribe_batch(groups[0][:1], dec_id) if dec_id != 2 else model.transcribe_batch_aed(groups[0][:1], AED_PROMPT, AED_EOS, cfg.aed_max_gen_delta)
                b1_e2e = (time.perf_counter() - t0) / 5
                line["batch1"] = {"value": secs[0] * 5 / (bms * 1e-3), "unit": UNIT, "ms_per_step": bms / 5,
                                  "e2e": secs[0] / b1_e2e, "workload": f"1 x {secs[0]:g} s per step"}
            for bh in bh2:
                model.batch_free(bh)
            line["roofline_hbm"] = hbm_roofline(pkg, synth, cfg, peaks)
            try:
                line["a8"] = a8_section(args, pkg, synth, torch, groups, dec_id, audio_s, peaks)
            except pkg.BackendError as e:
                line["a8"] = {"unavailable": str(e)}
        if world == 1 and not args.no_cpu_baseline:
            cb, rep = cpu_baseline(args, cfg, tensors, synth, model)
            if rep is not None:       # the reference decoded the same utterance as item `sample_index` of this rank
                u = args.sample_index
                ref_t, ref_f = rep.pop("_ref_tokens"), rep.pop("_ref_frames")
                rep["utterance"] = u
                rep["tokens"]["timed_batch_item_identical"] = ref_t == res[u][0] and (ref_f is None or ref_f == res[u][1])
                rep["recipe"] = "baseline: linears ~ N(0, 0.02), seed 0 (the timed model)"
                line["parity"] = rep
                if not args.no_diverse:
                    line["parity_diverse"] = parity_diverse(args, pkg, synth, args.seconds)
            line["cpu_baseline"] = cb
        else:
            line["cpu_baseline"] = {"value": None, "unit": UNIT, "cores": os.cpu_count(), "kind": "reference",
                                    "sample": "timed at N=1 only"}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
