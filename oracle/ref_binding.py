"""ctypes access to the UNMODIFIED reference compiled into
oracle/_ref/libmynah_ref.so — TEST INFRASTRUCTURE ONLY (see oracle/Makefile,
oracle/ref_harness.c). Used to pin the numpy oracle, to generate the golden
fixtures under tests/golden/, and as the timed CPU baseline of the benchmark.
Never imported by the product.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_ref", "libmynah_ref.so")

c_fp = C.POINTER(C.c_float)
c_ip = C.POINTER(C.c_int)


def available() -> bool:
    return os.path.exists(LIB_PATH)


_lib = None
CUDA_LIB_PATH = os.path.join(_HERE, "_ref", "libmynah_ref_cuda.so")      # `make -C oracle cuda`: the reference on the B200 backend


def lib():
    global _lib
    if _lib is None:
        _lib = load(LIB_PATH)
    return _lib


_cuda_lib = None


def cuda_lib():
    """The reference with integration/*.patch applied, compiled with -DMYNAH_ASR_CUDA and linked against
    libmynah_b200.so: its own mynah_asr_set_backend("cuda") routes the GEMMs and quantised products there."""
    global _cuda_lib
    if _cuda_lib is None:
        L = load(CUDA_LIB_PATH)
        L.mynah_asr_set_backend.argtypes = [C.c_char_p]
        L.mynah_asr_backend.restype = C.c_int
        _cuda_lib = L
    return _cuda_lib


def load(path):
    if True:
        L = C.CDLL(path)
        L.ref_open.restype = C.c_void_p
        L.ref_open.argtypes = [C.c_char_p, C.c_char_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                               C.c_int, C.c_int, c_ip, C.c_int]
        L.ref_close.argtypes = [C.c_void_p]
        L.ref_dims.argtypes = [C.c_void_p, c_ip]
        L.ref_free.argtypes = [C.c_void_p]
        L.ref_log_mel.restype = C.c_void_p
        L.ref_log_mel.argtypes = [C.c_void_p, c_fp, C.c_size_t, c_ip, c_ip]
        L.ref_subsampling.restype = C.c_void_p
        L.ref_subsampling.argtypes = [C.c_void_p, c_fp, C.c_int, C.c_int, c_ip]
        L.ref_pos_emb.argtypes = [C.c_void_p, C.c_int, c_fp]
        L.ref_encoder_layer.argtypes = [C.c_void_p, C.c_int, c_fp, C.c_int, c_fp, C.c_int, C.c_int]
        L.ref_encoder_post.argtypes = [C.c_void_p, c_fp, C.c_int, c_fp]
        L.ref_encoder_forward.restype = C.c_void_p
        L.ref_encoder_forward.argtypes = [C.c_void_p, c_fp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, c_ip]
        L.ref_encoder_forward_batch.argtypes = [C.c_void_p, C.POINTER(c_fp), c_ip, C.c_int, C.c_int, C.c_int,
                                                C.c_int, C.POINTER(C.c_void_p), c_ip]
        L.ref_encoder_forward_p.restype = C.c_void_p
        L.ref_encoder_forward_p.argtypes = [C.c_void_p, c_fp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, c_ip]
        L.ref_encoder_forward_batch_p.argtypes = [C.c_void_p, C.POINTER(c_fp), c_ip, C.c_int, C.c_int, c_ip, C.c_int,
                                                  C.c_int, C.POINTER(C.c_void_p), c_ip]
        L.ref_stream_step_p.argtypes = [C.c_void_p, c_fp, C.c_int, C.c_int, C.c_int, C.c_int, c_fp]
        L.ref_ctc_decode.argtypes = [C.c_void_p, c_fp, C.c_int, c_ip, c_ip, C.c_int]
        L.ref_greedy_decode.argtypes = [C.c_void_p, c_fp, C.c_int, c_ip, c_ip, C.c_int]
        L.ref_aed_open.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]
        L.ref_aed_decode.argtypes = [C.c_void_p, c_fp, C.c_int, c_ip, C.c_int, C.c_int, c_ip, C.c_int]
        L.ref_stream_open.restype = C.c_void_p
        L.ref_stream_open.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int]
        L.ref_stream_need.argtypes = [C.c_void_p]
        L.ref_stream_step.argtypes = [C.c_void_p, c_fp, C.c_int, C.c_int, C.c_int, c_fp]
        L.ref_stream_close.argtypes = [C.c_void_p]
        L.ref_qmat_mul_from_f32.argtypes = [c_fp, C.c_int, C.c_int, C.c_int, c_fp, c_fp, C.c_int]
        L.ref_align_ctc.argtypes = [c_fp, C.c_int, C.c_int, c_ip, C.c_int, C.c_int, c_ip, c_ip]
        L.ref_align_min_frames.argtypes = [c_ip, C.c_int]
        if hasattr(L, "ref_vad_open"):        # the planner shim is part of the plain build only
            L.ref_vad_open.restype = C.c_void_p
            L.ref_vad_open.argtypes = [C.c_char_p]
            L.ref_vad_close.argtypes = [C.c_void_p]
            L.ref_vad_reset.argtypes = [C.c_void_p]
            L.ref_vad_feed.restype = C.c_float
            L.ref_vad_feed.argtypes = [C.c_void_p, c_fp, C.c_size_t]
            L.ref_vad_speech_spans.argtypes = [C.c_void_p, c_fp, C.c_size_t, C.POINTER(C.c_longlong), C.c_int]
            L.ref_plan_segments.argtypes = [c_fp, C.c_size_t, C.c_int, C.c_double, C.c_void_p, C.POINTER(C.c_longlong), C.c_int]
        L.ingot_dequant.argtypes = [C.c_int, C.c_void_p, C.c_size_t, c_fp]
        L.ingot_quantize.argtypes = [C.c_int, c_fp, C.c_size_t, C.c_void_p]
    return L


def _fp(a):
    return a.ctypes.data_as(c_fp)


def _take(ptr, shape):
    """Copy a malloc'd float buffer returned by the reference, then free it."""
    n = int(np.prod(shape))
    out = np.ctypeslib.as_array(C.cast(ptr, c_fp), shape=(n,)).copy().reshape(shape)
    lib().ref_free(ptr)
    return out


def ggml_dequant(ggml_type: int, raw: np.ndarray, nelem: int) -> np.ndarray:
    raw = np.ascontiguousarray(raw, np.uint8)
    out = np.empty(nelem, np.float32)
    rc = lib().ingot_dequant(ggml_type, raw.ctypes.data, nelem, _fp(out))
    assert rc == 0
    return out


def ggml_quantize(ggml_type: int, w: np.ndarray, nbytes: int) -> np.ndarray:
    w = np.ascontiguousarray(w, np.float32).reshape(-1)
    out = np.zeros(nbytes, np.uint8)
    rc = lib().ingot_quantize(ggml_type, _fp(w), w.size, out.ctypes.data)
    assert rc == 0
    return out


class RefVad:
    """mynah_asr_vad over a model directory (mynah.json + model.safetensors), src/vad.c."""

    def __init__(self, model_dir):
        self.h = lib().ref_vad_open(model_dir.encode())
        if not self.h:
            raise RuntimeError("reference failed to open the VAD at " + model_dir)

    def close(self):
        if self.h:
            lib().ref_vad_close(self.h)
            self.h = None

    def probs(self, samples, frame=512):
        samples = np.ascontiguousarray(samples, np.float32)
        lib().ref_vad_reset(self.h)
        out = []
        for o in range(0, samples.size, frame):
            piece = np.ascontiguousarray(samples[o:o + frame])
            out.append(float(lib().ref_vad_feed(self.h, _fp(piece), piece.size)))
        return out

    def speech_spans(self, samples):
        samples = np.ascontiguousarray(samples, np.float32)
        cap = samples.size // 1024 + 2
        buf = (C.c_longlong * (2 * cap))()
        k = lib().ref_vad_speech_spans(self.h, _fp(samples), samples.size, buf, cap)
        assert k >= 0
        return [(int(buf[2 * i]), int(buf[2 * i + 1])) for i in range(k)]


def plan_segments(samples, sample_rate, seg_sec, vad=None):
    """plan_segments (src/mynah_asr.c:1287-1323; the VAD plan :1216-1280 when vad is a RefVad): [(offset, length)]."""
    samples = np.ascontiguousarray(samples, np.float32)
    cap = max(16, int(samples.size / max(sample_rate * 1.0, 1)) + 16)
    buf = (C.c_longlong * (2 * cap))()
    k = lib().ref_plan_segments(_fp(samples), samples.size, sample_rate, seg_sec, vad.h if vad else None, buf, cap)
    assert 0 <= k <= cap
    return [(int(buf[2 * i]), int(buf[2 * i + 1])) for i in range(k)]


def align_ctc(scores, tokens, blank):
    """mynah_asr_align_ctc (src/align.c): (rc, t0, t1) for scores [T, V] and a label sequence."""
    scores = np.ascontiguousarray(scores, np.float32)
    tk = np.ascontiguousarray(tokens, np.int32)
    t0 = np.full(max(tk.size, 1), -1, np.int32)
    t1 = np.full(max(tk.size, 1), -1, np.int32)
    rc = lib().ref_align_ctc(_fp(scores), scores.shape[0], scores.shape[1], tk.ctypes.data_as(c_ip), tk.size, blank,
                             t0.ctypes.data_as(c_ip), t1.ctypes.data_as(c_ip))
    return rc, t0[:tk.size].tolist(), t1[:tk.size].tolist()


def qmat_mul(w: np.ndarray, qtype: int, x: np.ndarray, library=None) -> np.ndarray:
    """The reference's mynah_asr_qmat_mul on W quantised by its own load-time
    quantiser (qtype 0 f32, 1 int8, 2 int4)."""
    w = np.ascontiguousarray(w, np.float32)
    x = np.ascontiguousarray(x, np.float32)
    out = np.empty((x.shape[0], w.shape[0]), np.float32)
    rc = (library or lib()).ref_qmat_mul_from_f32(_fp(w), w.shape[0], w.shape[1], qtype, _fp(x), _fp(out), x.shape[0])
    assert rc == 0
    return out


class RefModel:
    """The reference encoder/decoder over a safetensors file of f32 weights."""

    def __init__(self, weights_path, mel_path=None, *, quant=0, causal=-1, xscaling=0, n_mels=80,
                 normalize=1, blank=0, max_symbols=10, durations=(), library=None):
        self.L = library or lib()
        d = (C.c_int * max(1, len(durations)))(*durations)
        self.h = self.L.ref_open(weights_path.encode(), mel_path.encode() if mel_path else None, quant, causal,
                                xscaling, n_mels, normalize, blank, max_symbols, d if durations else None,
                                len(durations))
        if not self.h:
            raise RuntimeError("reference failed to open " + weights_path)
        dims = (C.c_int * 8)()
        self.L.ref_dims(self.h, dims)
        (self.d_model, self.n_layers, self.n_heads, self.ffn_dim, self.conv_k, self.d_out, self.causal,
         self.channels) = list(dims)
        self.n_mels = n_mels

    def close(self):
        if self.h:
            self.L.ref_close(self.h)
            self.h = None

    def log_mel(self, audio):
        audio = np.ascontiguousarray(audio, np.float32)
        T, v = C.c_int(), C.c_int()
        p = self.L.ref_log_mel(self.h, _fp(audio), audio.size, C.byref(T), C.byref(v))
        assert p
        return _take(p, (T.value, self.n_mels)), v.value

    def subsampling(self, feats):
        feats = np.ascontiguousarray(feats, np.float32)
        t = C.c_int()
        p = self.L.ref_subsampling(self.h, _fp(feats), feats.shape[0], feats.shape[1], C.byref(t))
        assert p
        return _take(p, (t.value, self.d_model))

    def pos_emb(self, T):
        pe = np.empty((2 * T - 1, self.d_model), np.float32)
        self.L.ref_pos_emb(self.h, T, _fp(pe))
        return pe

    def encoder_layer(self, li, x, pe, left=-1, right=-1):
        x = np.ascontiguousarray(x, np.float32).copy()
        rc = self.L.ref_encoder_layer(self.h, li, _fp(x), x.shape[0], _fp(pe), left, right)
        assert rc == 0
        return x

    def encoder_post(self, x):
        x = np.ascontiguousarray(x, np.float32)
        out = np.empty((x.shape[0], self.d_out), np.float32)
        self.L.ref_encoder_post(self.h, _fp(x), x.shape[0], _fp(out))
        return out

    def encoder_forward(self, feats, left=-1, right=-1, raw=False, prompt_id=0):
        feats = np.ascontiguousarray(feats, np.float32)
        t = C.c_int()
        if prompt_id and not raw:
            p = self.L.ref_encoder_forward_p(self.h, _fp(feats), feats.shape[0], feats.shape[1], prompt_id, left, right,
                                            C.byref(t))
        else:
            p = self.L.ref_encoder_forward(self.h, _fp(feats), feats.shape[0], feats.shape[1], left, right, int(raw),
                                          C.byref(t))
        assert p
        return _take(p, (t.value, self.d_model if raw else self.d_out))

    def encoder_forward_batch(self, feats_list, left=-1, right=-1, prompt_ids=None):
        B = len(feats_list)
        fl = [np.ascontiguousarray(f, np.float32) for f in feats_list]
        ptrs = (c_fp * B)(*[_fp(f) for f in fl])
        tm = (C.c_int * B)(*[f.shape[0] for f in fl])
        outs = (C.c_void_p * B)()
        touts = (C.c_int * B)()
        if prompt_ids is not None:
            pid = (C.c_int * B)(*prompt_ids)
            rc = self.L.ref_encoder_forward_batch_p(self.h, ptrs, tm, B, fl[0].shape[1], pid, left, right, outs, touts)
        else:
            rc = self.L.ref_encoder_forward_batch(self.h, ptrs, tm, B, fl[0].shape[1], left, right, outs, touts)
        assert rc == 0
        return [_take(outs[b], (touts[b], self.d_out)) for b in range(B)]

    def _decode(self, fn, enc, cap):
        enc = np.ascontiguousarray(enc, np.float32)
        toks = np.zeros(cap, np.int32)
        frames = np.zeros(cap, np.int32)
        n = fn(self.h, _fp(enc), enc.shape[0], toks.ctypes.data_as(c_ip), frames.ctypes.data_as(c_ip), cap)
        assert n >= 0
        return toks[:n].tolist(), frames[:n].tolist()

    def ctc_decode(self, enc):
        return self._decode(self.L.ref_ctc_decode, enc, enc.shape[0])

    def greedy_decode(self, enc, max_symbols=10):
        return self._decode(self.L.ref_greedy_decode, enc, enc.shape[0] * max_symbols)

    def aed_open(self, n_layers, n_heads, max_seq, max_gen_delta, quant=0):
        if self.L.ref_aed_open(self.h, n_layers, n_heads, max_seq, max_gen_delta, quant) != 0:
            raise RuntimeError("reference: AED weights missing or incomplete")

    def aed_decode(self, enc, prompt, eos, cap):
        """mynah_asr_aed_decode (src/decoder_aed.c:139-232): generated tokens, prompt and EOS excluded."""
        enc = np.ascontiguousarray(enc, np.float32)
        pr = np.ascontiguousarray(prompt, np.int32)
        out = np.zeros(max(cap, 1), np.int32)
        n = self.L.ref_aed_decode(self.h, _fp(enc), enc.shape[0], pr.ctypes.data_as(C.POINTER(C.c_int)), pr.size, eos,
                                 out.ctypes.data_as(C.POINTER(C.c_int)), cap)
        assert n >= 0
        return out[:n].copy()

    def stream_encode(self, mel, left, right, prompt_id=0):
        """Feed valid mel frames through the cache-aware streaming encoder in the
        exact chunk sizes it asks for; returns the concatenated [T, d_out]."""
        es = self.L.ref_stream_open(self.h, left, right, self.n_mels)
        assert es
        outs, pos, T = [], 0, mel.shape[0]
        buf = np.empty((right + 3, self.d_out), np.float32)
        while pos < T:
            need = self.L.ref_stream_need(es)
            chunk = np.ascontiguousarray(mel[pos:pos + need], np.float32)
            last = int(pos + need >= T)
            q = self.L.ref_stream_step_p(es, _fp(chunk), chunk.shape[0], mel.shape[1], prompt_id, last, _fp(buf))
            if q <= 0:
                break
            outs.append(buf[:q].copy())
            pos += need
        self.L.ref_stream_close(es)
        return np.concatenate(outs, 0) if outs else np.zeros((0, self.d_out), np.float32)
