"""mynah-asr_b200 — host-side mirror of the reference's hot-path interface over the
B200 CUDA library (include/mynah_b200.h).

The product is the C-ABI shared library built from csrc/; this module is the thin
ctypes binding tests and the benchmark use — the same kind of binding the
reference ships for its own library (bindings/python/mynah_asr.py). Function and
argument names follow the reference: qmat_mul, log_mel, subsampling_forward,
encoder_layer, encoder_forward(_raw/_batch), ctc_decode, greedy_decode.

There is no CPU path here: if the CUDA library is missing or no sm_100 device is
present, loading fails loudly.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libmynah_b200.so")

F32, MYNAH_Q8, MYNAH_Q4 = 0, 1, 2
GGML_Q4_0, GGML_Q8_0, GGML_Q4_K, GGML_Q6_K = 102, 108, 112, 114
A16, A8, FAST, SCALAR, MMA_SYNC, FEW_ROWS = 0, 1, 2, 4, 8, 16

c_fp = C.POINTER(C.c_float)
c_ip = C.POINTER(C.c_int)


class Config(C.Structure):
    _fields_ = [("n_mels", C.c_int), ("n_fft", C.c_int), ("win_length", C.c_int), ("hop_length", C.c_int),
                ("preemphasis", C.c_double), ("log_zero_guard", C.c_double), ("normalize_per_feature", C.c_int),
                ("causal", C.c_int), ("xscaling", C.c_int), ("left_ctx", C.c_int), ("right_ctx", C.c_int),
                ("blank_id", C.c_int), ("max_symbols", C.c_int), ("n_durations", C.c_int),
                ("durations", C.c_int * 16), ("strict", C.c_int), ("attn_impl", C.c_int), ("aed_heads", C.c_int), ("a8", C.c_int)]


class VadConfig(C.Structure):
    _fields_ = [("frame_samples", C.c_int), ("context_samples", C.c_int), ("reflect_pad", C.c_int), ("n_fft", C.c_int),
                ("hop_length", C.c_int), ("n_bins", C.c_int), ("lstm_hidden", C.c_int), ("n_enc", C.c_int),
                ("enc_channels", C.c_int * 8), ("enc_kernels", C.c_int * 8), ("enc_strides", C.c_int * 8),
                ("enc_pads", C.c_int * 16), ("threshold", C.c_double), ("neg_threshold", C.c_double),
                ("min_speech_ms", C.c_int), ("min_silence_ms", C.c_int), ("speech_pad_ms", C.c_int)]


class BackendError(RuntimeError):
    pass


class StreamGroup:
    """n streams advancing in lock step through the cache-aware streaming encoder."""

    def __init__(self, model, handle, n, q):
        self.model, self.h, self.n, self.q = model, handle, n, q

    def need(self):
        return lib().mynah_b200_stream_need(self.h)

    def set_prompts(self, prompt_ids):
        """one prompt id per stream (prompt-conditioned encoders), before the first step"""
        assert len(prompt_ids) == self.n
        if lib().mynah_b200_stream_set_prompts(self.h, (C.c_int * self.n)(*prompt_ids)) != 0:
            raise BackendError("stream_set_prompts: " + _err())

    def step(self, mel, is_last=False):
        """mel [n, n_mel, n_mels] -> [n, q, d_out]"""
        mel = np.ascontiguousarray(mel, np.float32)
        assert mel.ndim == 3 and mel.shape[0] == self.n
        out = np.empty((self.n, self.q + 2, self.model.d_out), np.float32)
        q = lib().mynah_b200_stream_step(self.h, _fp(mel), mel.shape[1], int(is_last), _fp(out))
        if q < 0:
            raise BackendError("stream_step: " + _err())
        return out.reshape(-1)[:self.n * q * self.model.d_out].reshape(self.n, q, self.model.d_out).copy()

    def mel_feed(self, audio, finish=False, cap_frames=4096):
        """audio [n, samples] -> the log-mel frames that became ready, [n, frames, n_mels]"""
        audio = np.ascontiguousarray(audio, np.float32)
        assert audio.ndim == 2 and audio.shape[0] == self.n
        out = np.empty((self.n * cap_frames * self.model.n_mels,), np.float32)
        k = lib().mynah_b200_stream_mel_feed(self.h, _fp(audio), audio.shape[1], int(finish), _fp(out), cap_frames)
        if k < 0:
            raise BackendError("stream_mel_feed: " + _err())
        return out[:self.n * k * self.model.n_mels].reshape(self.n, k, self.model.n_mels).copy()

    def step_decode(self, mel, is_last=False):
        """mel [n, n_mel, n_mels] -> per stream (tokens, absolute frames) emitted on this chunk"""
        mel = np.ascontiguousarray(mel, np.float32)
        assert mel.ndim == 3 and mel.shape[0] == self.n
        tk, fr, nt = (C.c_void_p * self.n)(), (C.c_void_p * self.n)(), (C.c_int * self.n)()
        q = lib().mynah_b200_stream_step_decode(self.h, _fp(mel), mel.shape[1], int(is_last), tk, fr, nt)
        if q < 0:
            raise BackendError("stream_step_decode: " + _err())
        return [(_take_i32(tk[s], nt[s]), _take_i32(fr[s], nt[s])) for s in range(self.n)]

    def close(self):
        if self.h:
            lib().mynah_b200_stream_close(self.h)
            self.h = None


_lib = None


def lib():
    """Loads the CUDA library. Raises if it has not been built — never falls back."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise BackendError(f"{LIB_PATH} is missing: build it with `python __graft_entry__.py` "
                           "(or mynah-asr_b200/build.py); there is no CPU fallback")
    L = C.CDLL(LIB_PATH)
    vp, ci, cf = C.c_void_p, C.c_int, C.c_float
    L.mynah_b200_last_error.restype = C.c_char_p
    L.mynah_b200_available.restype = ci
    L.mynah_b200_select_device.argtypes = [ci]
    L.mynah_b200_launch_count.restype = C.c_longlong
    L.mynah_b200_launch_count.argtypes = [ci]
    L.mynah_b200_config_default.argtypes = [C.POINTER(Config)]
    L.mynah_b200_gemm_wt.argtypes = [c_fp, c_fp, c_fp, ci, ci, ci]
    L.mynah_asr_cuda_gemm_wt.argtypes = [c_fp, c_fp, c_fp, ci, ci, ci]
    L.mynah_b200_qgemm.argtypes = [vp, ci, c_fp, ci, ci, c_fp, c_fp, ci, ci]
    L.mynah_b200_weights_evict.restype = None
    L.mynah_b200_qmat_create.restype = vp
    L.mynah_b200_qmat_create.argtypes = [ci, vp, c_fp, ci, ci]
    L.mynah_b200_qmat_free.argtypes = [vp]
    L.mynah_b200_qmat_mul.argtypes = [vp, c_fp, c_fp, ci, ci]
    L.mynah_b200_qmat_block_dots.argtypes = [vp, c_fp, ci, C.POINTER(C.c_int32), c_fp, c_fp]
    L.mynah_b200_qmat_dequant.argtypes = [vp, c_fp]
    L.mynah_b200_qmat_mul_a8_static.argtypes = [vp, vp, vp, ci]
    L.mynah_b200_qmat_time.restype = C.c_double
    L.mynah_b200_qmat_time.argtypes = [vp, ci, ci, ci]
    L.mynah_b200_profile_begin.argtypes = [vp]
    L.mynah_b200_profile_end.argtypes = [vp, C.POINTER(C.c_double), C.POINTER(C.c_double), C.POINTER(C.c_longlong), ci]
    L.mynah_b200_aed_decode.argtypes = [vp, c_fp, ci, c_ip, ci, ci, c_ip, ci]
    L.mynah_b200_aed_decode_batch.argtypes = [vp, C.POINTER(c_fp), c_ip, ci, C.POINTER(C.POINTER(C.c_int)), c_ip, ci, c_ip,
                                              C.POINTER(C.c_void_p), c_ip]
    L.mynah_b200_transcribe_batch_aed.argtypes = [vp, C.POINTER(c_fp), C.POINTER(C.c_size_t), ci, c_ip, ci, ci, ci,
                                                  C.POINTER(C.c_void_p), c_ip]
    L.mynah_b200_batch_set_aed.argtypes = [vp, c_ip, ci, ci, ci]
    L.mynah_b200_batch_set_aed.restype = None
    L.mynah_b200_stream_open.restype = vp
    L.mynah_b200_stream_open.argtypes = [vp, ci, ci, ci]
    L.mynah_b200_stream_close.argtypes = [vp]
    L.mynah_b200_stream_close.restype = None
    L.mynah_b200_stream_need.argtypes = [vp]
    L.mynah_b200_stream_step.argtypes = [vp, c_fp, ci, ci, c_fp]
    L.mynah_b200_stream_step_device.argtypes = [vp, vp, ci, ci, vp]
    L.mynah_b200_stream_mel_feed.argtypes = [vp, c_fp, ci, ci, c_fp, ci]
    L.mynah_b200_stream_step_decode.argtypes = [vp, c_fp, ci, ci, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), c_ip]
    L.mynah_b200_profile_bytes.argtypes = [vp, C.POINTER(C.c_double), ci]
    L.mynah_b200_decoder_clocks.argtypes = [vp, C.POINTER(C.c_longlong)]
    L.mynah_b200_model_new.restype = vp
    L.mynah_b200_model_new.argtypes = [C.POINTER(Config)]
    L.mynah_b200_model_add_tensor.argtypes = [vp, C.c_char_p, ci, C.POINTER(C.c_int64), ci, vp]
    L.mynah_b200_model_set_mel.argtypes = [vp, c_fp, c_fp]
    L.mynah_b200_model_finalize.argtypes = [vp]
    L.mynah_b200_model_free.argtypes = [vp]
    L.mynah_b200_model_set_strict.argtypes = [vp, ci]
    L.mynah_b200_model_load.restype = vp
    L.mynah_b200_model_load.argtypes = [C.c_char_p, C.c_char_p, C.POINTER(Config), ci]
    L.mynah_b200_model_load_stats.argtypes = [vp, C.POINTER(C.c_double), C.POINTER(C.c_double), C.POINTER(C.c_double)]
    L.mynah_b200_model_set_max_contexts.argtypes = [vp, ci]
    L.mynah_b200_model_dims.argtypes = [vp, c_ip]
    L.mynah_b200_model_stream.restype = vp
    L.mynah_b200_model_stream.argtypes = [vp]
    L.mynah_b200_log_mel.restype = vp
    L.mynah_b200_log_mel.argtypes = [vp, c_fp, C.c_size_t, c_ip, c_ip]
    L.mynah_b200_subsampling_forward.restype = vp
    L.mynah_b200_subsampling_forward.argtypes = [vp, c_fp, ci, ci, c_ip]
    L.mynah_b200_encoder_layer.argtypes = [vp, ci, c_fp, ci, ci, ci]
    L.mynah_b200_encoder_forward.restype = vp
    L.mynah_b200_encoder_forward.argtypes = [vp, c_fp, ci, ci, ci, ci, ci, c_ip]
    L.mynah_b200_encoder_forward_raw.restype = vp
    L.mynah_b200_encoder_forward_raw.argtypes = [vp, c_fp, ci, ci, ci, ci, c_ip]
    L.mynah_b200_encoder_forward_batch.argtypes = [vp, C.POINTER(c_fp), c_ip, ci, ci, c_ip, ci, ci,
                                                   C.POINTER(vp), c_ip]
    L.mynah_b200_ctc_decode.argtypes = [vp, c_fp, ci, c_ip, c_ip, ci]
    L.mynah_b200_greedy_decode.argtypes = [vp, c_fp, ci, c_ip, c_ip, ci]
    L.mynah_b200_transcribe_batch.argtypes = [vp, C.POINTER(c_fp), C.POINTER(C.c_size_t), ci, ci, C.POINTER(vp),
                                              C.POINTER(vp), c_ip]
    L.mynah_b200_transcribe_batch_prompts.argtypes = [vp, C.POINTER(c_fp), C.POINTER(C.c_size_t), ci, c_ip, ci, C.POINTER(vp),
                                                      C.POINTER(vp), c_ip]
    L.mynah_b200_stream_set_prompts.argtypes = [vp, c_ip]
    L.mynah_b200_batch_set_prompts.argtypes = [vp, c_ip]
    L.mynah_b200_batch_set_prompts.restype = None
    L.mynah_b200_qmat_sync.argtypes = [vp]
    L.mynah_b200_align_ctc.argtypes = [c_fp, ci, ci, c_ip, ci, ci, c_ip, c_ip]
    L.mynah_b200_align_min_frames.argtypes = [c_ip, ci]
    L.mynah_b200_ctc_align.argtypes = [vp, c_fp, ci, c_ip, ci, c_ip, c_ip]
    L.mynah_b200_vad_new.restype = vp
    L.mynah_b200_vad_new.argtypes = [C.POINTER(VadConfig), c_fp, C.POINTER(c_fp), C.POINTER(c_fp), c_fp, c_fp, c_fp, c_fp, c_fp, cf]
    L.mynah_b200_vad_free.argtypes = [vp]
    L.mynah_b200_vad_free.restype = None
    L.mynah_b200_vad_probs.argtypes = [vp, c_fp, C.c_size_t, c_fp, ci]
    L.mynah_b200_vad_speech_spans.argtypes = [vp, c_fp, C.c_size_t, C.POINTER(C.c_longlong), ci]
    L.mynah_b200_plan_segments.argtypes = [vp, c_fp, C.c_size_t, ci, C.c_double, C.POINTER(C.c_longlong), ci]
    L.mynah_b200_batch_upload.restype = vp
    L.mynah_b200_batch_upload.argtypes = [vp, C.POINTER(c_fp), C.POINTER(C.c_size_t), ci]
    L.mynah_b200_batch_run.argtypes = [vp, vp, ci]
    L.mynah_b200_batch_fetch.argtypes = [vp, vp, C.POINTER(vp), C.POINTER(vp), c_ip]
    L.mynah_b200_batch_free.argtypes = [vp]
    _lib = L
    return L


_libc = C.CDLL(None)
_libc.free.argtypes = [C.c_void_p]


def _err() -> str:
    return lib().mynah_b200_last_error().decode(errors="replace")


def _check(rc, what):
    if rc != 0:
        raise BackendError(f"{what}: {_err()}")


def _fp(a):
    return a.ctypes.data_as(c_fp)


def _take_f32(ptr, shape):
    if not ptr:
        raise BackendError(_err())
    n = int(np.prod(shape))
    out = np.ctypeslib.as_array(C.cast(ptr, c_fp), shape=(max(n, 1),))[:n].copy().reshape(shape)
    _libc.free(ptr)
    return out


def _take_i32(ptr, n):
    out = np.ctypeslib.as_array(C.cast(ptr, c_ip), shape=(max(n, 1),))[:n].copy()
    _libc.free(ptr)
    return out.tolist()


def available() -> bool:
    return bool(lib().mynah_b200_available())


def launch_count(reset: bool = False) -> int:
    return int(lib().mynah_b200_launch_count(int(reset)))


def gemm_wt(x, w):
    """out[T,n] = x[T,k] @ W[n,k]^T (mynah_asr_gemm_wt, src/backend.c:68-81)."""
    x = np.ascontiguousarray(x, np.float32); w = np.ascontiguousarray(w, np.float32)
    out = np.empty((x.shape[0], w.shape[0]), np.float32)
    _check(lib().mynah_b200_gemm_wt(_fp(x), _fp(w), _fp(out), x.shape[0], w.shape[0], w.shape[1]), "gemm_wt")
    return out


def cuda_gemm_wt(x, w):
    """The reference's hook under its own name (mynah_asr_cuda_gemm_wt, src/cuda_gemm.cu:144-190): `w` must be a
    C-contiguous float32 array that stays alive and unchanged; it is uploaded on the first call with this address."""
    assert w.dtype == np.float32 and w.flags.c_contiguous
    x = np.ascontiguousarray(x, np.float32)
    out = np.empty((x.shape[0], w.shape[0]), np.float32)
    if lib().mynah_asr_cuda_gemm_wt(_fp(x), _fp(w), _fp(out), x.shape[0], w.shape[0], w.shape[1]) != 0:
        raise BackendError("mynah_asr_cuda_gemm_wt: " + _err())
    return out


def qgemm(raw, fmt, n, k, x, flags=A16, scales=None):
    """mynah_b200_qgemm: quantised operand found by the address of `raw` (a uint8 array the caller keeps alive)."""
    assert raw.dtype == np.uint8 and raw.flags.c_contiguous
    x = np.ascontiguousarray(x, np.float32)
    out = np.empty((x.shape[0], n), np.float32)
    sc = None if scales is None else _fp(scales)
    _check(lib().mynah_b200_qgemm(raw.ctypes.data, fmt, sc, n, k, _fp(x), _fp(out), x.shape[0], flags), "qgemm")
    return out


def weights_evict():
    lib().mynah_b200_weights_evict()


def weights_resident() -> int:
    return int(lib().mynah_b200_weights_resident())


def align_ctc(scores, tokens, blank):
    """mynah_asr_align_ctc (src/align.c) on the device: (rc, t0, t1) for scores [T, V] and a label sequence."""
    scores = np.ascontiguousarray(scores, np.float32)
    n = len(tokens)
    tk = (C.c_int * max(n, 1))(*tokens)
    t0, t1 = (C.c_int * max(n, 1))(), (C.c_int * max(n, 1))()
    rc = lib().mynah_b200_align_ctc(_fp(scores), scores.shape[0], scores.shape[1], tk, n, blank, t0, t1)
    return rc, list(t0[:n]), list(t1[:n])


def align_min_frames(tokens):
    return lib().mynah_b200_align_min_frames((C.c_int * max(len(tokens), 1))(*tokens), len(tokens))


class Vad:
    """Silero-style voice activity model on the device (mynah_asr_vad, src/vad.h): cfg = the "vad" section of the
    model's mynah.json, tensors = {name: float32 array} with the names of its model.safetensors."""

    def __init__(self, cfg, tensors):
        c = VadConfig()
        for k in ("frame_samples", "context_samples", "reflect_pad", "n_fft", "hop_length", "n_bins", "lstm_hidden",
                  "min_speech_ms", "min_silence_ms", "speech_pad_ms"):
            setattr(c, k, int(cfg[k]))
        c.threshold, c.neg_threshold = float(cfg["threshold"]), float(cfg["neg_threshold"])
        ne = len(cfg["encoder_strides"])
        c.n_enc = ne
        for i in range(ne):
            c.enc_channels[i], c.enc_kernels[i], c.enc_strides[i] = cfg["encoder_channels"][i], cfg["encoder_kernels"][i], cfg["encoder_strides"][i]
            c.enc_pads[2 * i], c.enc_pads[2 * i + 1] = cfg["encoder_pads"][i]
        t = {k: np.ascontiguousarray(v, np.float32) for k, v in tensors.items()}
        self._keep = t
        ew = (c_fp * ne)(*[_fp(t[f"encoder.{i}.reparam_conv.weight"]) for i in range(ne)])
        eb = (c_fp * ne)(*[_fp(t[f"encoder.{i}.reparam_conv.bias"]) for i in range(ne)])
        self.frame = c.frame_samples
        self.h = lib().mynah_b200_vad_new(C.byref(c), _fp(t["stft.forward_basis_buffer"]), ew, eb, _fp(t["decoder.rnn.weight_ih"]),
                                          _fp(t["decoder.rnn.weight_hh"]), _fp(t["decoder.rnn.bias_ih"]), _fp(t["decoder.rnn.bias_hh"]),
                                          _fp(t["decoder.decoder.2.weight"]), float(t["decoder.decoder.2.bias"].reshape(-1)[0]))
        if not self.h:
            raise BackendError("vad_new: " + _err())

    def close(self):
        if getattr(self, "h", None):
            lib().mynah_b200_vad_free(self.h)
            self.h = None

    __del__ = close

    def probs(self, samples):
        s = np.ascontiguousarray(samples, np.float32)
        cap = s.size // self.frame + 2
        out = np.empty(cap, np.float32)
        k = lib().mynah_b200_vad_probs(self.h, _fp(s), s.size, _fp(out), cap)
        if k < 0:
            raise BackendError("vad_probs: " + _err())
        return out[:k].copy()

    def speech_spans(self, samples):
        s = np.ascontiguousarray(samples, np.float32)
        cap = s.size // (2 * self.frame) + 2
        buf = (C.c_longlong * (2 * cap))()
        k = lib().mynah_b200_vad_speech_spans(self.h, _fp(s), s.size, buf, cap)
        if k < 0:
            raise BackendError("vad_speech_spans: " + _err())
        return [(int(buf[2 * i]), int(buf[2 * i + 1])) for i in range(k)]


def plan_segments(samples, sample_rate, seg_sec, vad=None):
    """plan_segments (src/mynah_asr.c:1287-1323) with the signal on the device: [(offset, length)]."""
    s = np.ascontiguousarray(samples, np.float32)
    cap = max(16, int(s.size / max(sample_rate, 1)) + 16)
    buf = (C.c_longlong * (2 * cap))()
    k = lib().mynah_b200_plan_segments(vad.h if vad else None, _fp(s), s.size, sample_rate, seg_sec, buf, cap)
    if k < 0:
        raise BackendError("plan_segments: " + _err())
    return [(int(buf[2 * i]), int(buf[2 * i + 1])) for i in range(k)]


class QMat:
    """Resident quantised weight matrix [n,k] (mynah_asr_qmat, src/qmat.h:39-47)."""

    def __init__(self, fmt, data, n, k, scales=None):
        self._raw = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        self._scales = None if scales is None else np.ascontiguousarray(scales, np.float32)
        self.n, self.k, self.fmt = n, k, fmt
        self.h = lib().mynah_b200_qmat_create(fmt, self._raw.ctypes.data,
                                              None if self._scales is None else _fp(self._scales), n, k)
        if not self.h:
            raise BackendError("qmat_create: " + _err())

    def close(self):
        if self.h:
            lib().mynah_b200_qmat_free(self.h)
            self.h = None

    __del__ = close

    def mul(self, x, flags=A16):
        """out[T,n] = x[T,k] @ W^T (mynah_asr_qmat_mul, src/qmat.c:503-651)."""
        x = np.ascontiguousarray(x, np.float32)
        out = np.empty((x.shape[0], self.n), np.float32)
        _check(lib().mynah_b200_qmat_mul(self.h, _fp(x), _fp(out), x.shape[0], flags), "qmat_mul")
        return out

    def mul_a8_static(self, x_dev_ptr: int, out_dev_ptr: int, T: int):
        """A8 product on caller-owned DEVICE buffers without any device allocation: the
        scratch is a fixed array inside the library (T <= 16, k <= 8192). For hosts that
        may not call cudaMalloc while running. Synchronous."""
        _check(lib().mynah_b200_qmat_mul_a8_static(self.h, x_dev_ptr, out_dev_ptr, T), "qmat_mul_a8_static")

    def block_dots(self, x):
        x = np.ascontiguousarray(x, np.float32)
        T = x.shape[0]
        dots = np.empty((T, self.n, self.k // 32), np.int32)
        sx = np.empty(T, np.float32)
        out = np.empty((T, self.n), np.float32)
        _check(lib().mynah_b200_qmat_block_dots(self.h, _fp(x), T, dots.ctypes.data_as(C.POINTER(C.c_int32)),
                                                _fp(sx), _fp(out)), "qmat_block_dots")
        return dots, sx, out

    def dequant(self):
        wd = np.empty((self.n, self.k), np.float32)
        _check(lib().mynah_b200_qmat_dequant(self.h, _fp(wd)), "qmat_dequant")
        return wd

    def time_ms(self, T, flags=A16, iters=20):
        ms = lib().mynah_b200_qmat_time(self.h, T, flags, iters)
        if ms < 0:
            raise BackendError("qmat_time: " + _err())
        return ms


class Model:
    """Device-resident encoder + decoders built from named tensors
    (the weight side of mynah_asr_load_quant, src/mynah_asr.c:167-350)."""

    @staticmethod
    def _config(n_mels, causal=-1, xscaling=False, normalize=True, left=-1, right=-1, blank=0, max_symbols=10,
                durations=(), strict=True, attn_impl=0, aed_heads=8, a8=False):
        cfg = Config()
        lib().mynah_b200_config_default(C.byref(cfg))
        cfg.n_mels, cfg.causal, cfg.xscaling = n_mels, causal, int(xscaling)
        cfg.normalize_per_feature, cfg.left_ctx, cfg.right_ctx = int(normalize), left, right
        cfg.blank_id, cfg.max_symbols, cfg.n_durations = blank, max_symbols, len(durations)
        for i, d in enumerate(durations):
            cfg.durations[i] = d
        cfg.strict, cfg.attn_impl, cfg.aed_heads, cfg.a8 = int(strict), attn_impl, aed_heads, int(a8)
        return cfg

    @classmethod
    def load(cls, weights_path, mel_path=None, *, quant=0, n_mels, **kw):
        """The model straight from a safetensors or GGUF file (mynah_b200_model_load): the file is mapped and its
        tensors go to the device without a host-side decode. quant as in the reference's mynah_asr_load_quant."""
        self = cls.__new__(cls)
        self.cfg = cls._config(n_mels, **kw)
        self.h = lib().mynah_b200_model_load(weights_path.encode(), mel_path.encode() if mel_path else None,
                                             C.byref(self.cfg), quant)
        if not self.h:
            raise BackendError("model_load: " + _err())
        self._dims(n_mels, kw.get("max_symbols", 10))
        return self

    def load_stats(self):
        s, hb, db = C.c_double(), C.c_double(), C.c_double()
        lib().mynah_b200_model_load_stats(self.h, C.byref(s), C.byref(hb), C.byref(db))
        return {"seconds": s.value, "host_bytes": hb.value, "device_slab_bytes": db.value}

    def _dims(self, n_mels, max_symbols):
        dims = (C.c_int * 8)()
        lib().mynah_b200_model_dims(self.h, dims)
        (self.d_model, self.n_layers, self.n_heads, self.ffn_dim, self.conv_k, self.d_out, self.causal,
         self.channels) = list(dims)
        self.n_mels = n_mels
        self.max_symbols = max_symbols

    def __init__(self, tensors, *, n_mels, mel_fb=None, window=None, max_symbols=10, **kw):
        L = lib()
        cfg = self._config(n_mels, max_symbols=max_symbols, **kw)
        self.cfg = cfg
        self.h = L.mynah_b200_model_new(C.byref(cfg))
        if not self.h:
            raise BackendError("model_new: " + _err())
        keep = []
        for name, t in tensors.items():
            fmt = {0: F32, 2: GGML_Q4_0, 8: GGML_Q8_0, 12: GGML_Q4_K, 14: GGML_Q6_K, -8: MYNAH_Q8, -4: MYNAH_Q4}[t.ggml_type]
            shape = (C.c_int64 * len(t.shape))(*t.shape)
            raw = np.ascontiguousarray(t.raw)
            keep.append(raw)
            _check(L.mynah_b200_model_add_tensor(self.h, name.encode(), fmt, shape, len(t.shape), raw.ctypes.data),
                   "add_tensor " + name)
        if mel_fb is not None:
            fb = np.ascontiguousarray(mel_fb, np.float32); win = np.ascontiguousarray(window, np.float32)
            _check(L.mynah_b200_model_set_mel(self.h, _fp(fb), _fp(win)), "set_mel")
        _check(L.mynah_b200_model_finalize(self.h), "finalize")
        self._dims(n_mels, max_symbols)

    def close(self):
        if getattr(self, "h", None):
            lib().mynah_b200_model_free(self.h)
            self.h = None

    __del__ = close

    def set_max_contexts(self, n: int):
        """upper bound of calls that may run side by side on this model (one execution context each)"""
        _check(lib().mynah_b200_model_set_max_contexts(self.h, n), "model_set_max_contexts")

    def set_strict(self, strict: bool):
        """f32-grade three-product contractions (True) or a single fp16 product (False) for later calls"""
        _check(lib().mynah_b200_model_set_strict(self.h, int(strict)), "model_set_strict")

    def stream(self):
        return lib().mynah_b200_model_stream(self.h)

    PROFILE_CATEGORIES = ("gemm", "attention", "elementwise", "subsampling", "mel", "decode")

    def profile_begin(self):
        lib().mynah_b200_profile_begin(self.h)

    def profile_end(self):
        n = len(self.PROFILE_CATEGORIES)
        ms, fl, ln = (C.c_double * n)(), (C.c_double * n)(), (C.c_longlong * n)()
        _check(lib().mynah_b200_profile_end(self.h, ms, fl, ln, n), "profile_end")
        by = (C.c_double * n)()
        lib().mynah_b200_profile_bytes(self.h, by, n)
        return {c: {"ms": ms[i], "flops": fl[i], "launches": ln[i], "bytes": by[i]} for i, c in enumerate(self.PROFILE_CATEGORIES)}

    def decoder_clocks(self):
        out = (C.c_longlong * 8)()
        lib().mynah_b200_decoder_clocks(self.h, out)
        return list(out)

    def log_mel(self, audio):
        audio = np.ascontiguousarray(audio, np.float32)
        T, v = C.c_int(), C.c_int()
        p = lib().mynah_b200_log_mel(self.h, _fp(audio), audio.size, C.byref(T), C.byref(v))
        return _take_f32(p, (T.value, self.n_mels)), v.value

    def subsampling_forward(self, feats):
        feats = np.ascontiguousarray(feats, np.float32)
        t = C.c_int()
        p = lib().mynah_b200_subsampling_forward(self.h, _fp(feats), feats.shape[0], feats.shape[1], C.byref(t))
        return _take_f32(p, (t.value, self.d_model))

    def encoder_layer(self, li, x, left=-1, right=-1):
        x = np.ascontiguousarray(x, np.float32).copy()
        _check(lib().mynah_b200_encoder_layer(self.h, li, _fp(x), x.shape[0], left, right), "encoder_layer")
        return x

    def encoder_forward(self, feats, left=-1, right=-1, raw=False, prompt_id=0):
        feats = np.ascontiguousarray(feats, np.float32)
        t = C.c_int()
        if raw:
            p = lib().mynah_b200_encoder_forward_raw(self.h, _fp(feats), feats.shape[0], feats.shape[1], left, right,
                                                     C.byref(t))
        else:
            p = lib().mynah_b200_encoder_forward(self.h, _fp(feats), feats.shape[0], feats.shape[1], prompt_id, left, right,
                                                 C.byref(t))
        return _take_f32(p, (t.value, self.d_model if raw else self.d_out))

    def encoder_forward_batch(self, feats_list, left=-1, right=-1, prompt_ids=None):
        B = len(feats_list)
        fl = [np.ascontiguousarray(f, np.float32) for f in feats_list]
        ptrs = (c_fp * B)(*[_fp(f) for f in fl])
        tm = (C.c_int * B)(*[f.shape[0] for f in fl])
        pid = (C.c_int * B)(*(prompt_ids if prompt_ids is not None else [0] * B))
        outs = (C.c_void_p * B)()
        touts = (C.c_int * B)()
        _check(lib().mynah_b200_encoder_forward_batch(self.h, ptrs, tm, B, self.n_mels, pid, left, right, outs, touts),
               "encoder_forward_batch")
        return [_take_f32(outs[b], (touts[b], self.d_out)) for b in range(B)]

    def _decode(self, fn, enc, cap, what):
        enc = np.ascontiguousarray(enc, np.float32)
        toks = np.zeros(max(cap, 1), np.int32)
        frames = np.zeros(max(cap, 1), np.int32)
        n = fn(self.h, _fp(enc), enc.shape[0], toks.ctypes.data_as(c_ip), frames.ctypes.data_as(c_ip), cap)
        if n < 0:
            raise BackendError(what + ": " + _err())
        return toks[:n].tolist(), frames[:n].tolist()

    def ctc_decode(self, enc):
        return self._decode(lib().mynah_b200_ctc_decode, enc, enc.shape[0], "ctc_decode")

    def ctc_align(self, enc_raw, tokens):
        """first / last frame of every token's run: the model's CTC head over enc_raw, then forced alignment"""
        enc = np.ascontiguousarray(enc_raw, np.float32)
        n = len(tokens)
        tk = (C.c_int * n)(*tokens)
        t0, t1 = (C.c_int * n)(), (C.c_int * n)()
        _check(lib().mynah_b200_ctc_align(self.h, _fp(enc), enc.shape[0], tk, n, t0, t1), "ctc_align")
        return list(t0), list(t1)

    def greedy_decode(self, enc):
        return self._decode(lib().mynah_b200_greedy_decode, enc, enc.shape[0] * self.max_symbols, "greedy_decode")

    def aed_decode(self, enc, prompt, eos, cap):
        """mynah_asr_aed_decode: generated tokens, prompt and EOS excluded."""
        enc = np.ascontiguousarray(enc, np.float32)
        pr = (C.c_int * len(prompt))(*prompt)
        out = (C.c_int * max(cap, 1))()
        n = lib().mynah_b200_aed_decode(self.h, _fp(enc), enc.shape[0], pr, len(prompt), eos, out, cap)
        if n < 0:
            raise BackendError("aed_decode: " + _err())
        return np.array(out[:n], np.int32)

    def aed_decode_batch(self, encs, prompts, eos, caps):
        B = len(encs)
        el = [np.ascontiguousarray(e, np.float32) for e in encs]
        ep = (c_fp * B)(*[_fp(e) for e in el])
        Ts = (C.c_int * B)(*[e.shape[0] for e in el])
        pl = [(C.c_int * len(p))(*p) for p in prompts]
        pp = (C.POINTER(C.c_int) * B)(*[C.cast(p, C.POINTER(C.c_int)) for p in pl])
        npr = (C.c_int * B)(*[len(p) for p in prompts])
        cp = (C.c_int * B)(*caps)
        tk, nt = (C.c_void_p * B)(), (C.c_int * B)()
        _check(lib().mynah_b200_aed_decode_batch(self.h, ep, Ts, B, pp, npr, eos, cp, tk, nt), "aed_decode_batch")
        return [_take_i32(tk[b], nt[b]) for b in range(B)]

    def transcribe_batch_aed(self, audio_list, prompt, eos, max_gen_delta):
        B = len(audio_list)
        al, ptrs, ns = self._audio_args(audio_list)
        pr = (C.c_int * len(prompt))(*prompt)
        tk, nt = (C.c_void_p * B)(), (C.c_int * B)()
        _check(lib().mynah_b200_transcribe_batch_aed(self.h, ptrs, ns, B, pr, len(prompt), eos, max_gen_delta, tk, nt),
               "transcribe_batch_aed")
        return [_take_i32(tk[b], nt[b]) for b in range(B)]

    # ---- cache-aware streaming
    def stream_open(self, n_streams, left, right):
        g = lib().mynah_b200_stream_open(self.h, n_streams, left, right)
        if not g:
            raise BackendError("stream_open: " + _err())
        return StreamGroup(self, g, n_streams, right + 1)

    # ---- audio in, tokens out
    @staticmethod
    def _audio_args(audio_list):
        B = len(audio_list)
        al = [np.ascontiguousarray(a, np.float32) for a in audio_list]
        ptrs = (c_fp * B)(*[_fp(a) for a in al])
        ns = (C.c_size_t * B)(*[a.size for a in al])
        return al, ptrs, ns

    def transcribe_batch(self, audio_list, decoder=0, prompt_ids=None):
        B = len(audio_list)
        al, ptrs, ns = self._audio_args(audio_list)
        tk, fr, nt = (C.c_void_p * B)(), (C.c_void_p * B)(), (C.c_int * B)()
        pid = None if prompt_ids is None else (C.c_int * B)(*prompt_ids)
        _check(lib().mynah_b200_transcribe_batch_prompts(self.h, ptrs, ns, B, pid, decoder, tk, fr, nt), "transcribe_batch")
        return [(_take_i32(tk[b], nt[b]), _take_i32(fr[b], nt[b])) for b in range(B)]

    def batch_upload(self, audio_list):
        al, ptrs, ns = self._audio_args(audio_list)
        h = lib().mynah_b200_batch_upload(self.h, ptrs, ns, len(audio_list))
        if not h:
            raise BackendError("batch_upload: " + _err())
        return h

    def batch_set_aed(self, bh, prompt, eos, max_gen_delta):
        pr = (C.c_int * len(prompt))(*prompt)
        lib().mynah_b200_batch_set_aed(bh, pr, len(prompt), eos, max_gen_delta)

    def batch_run(self, bh, decoder=0):
        _check(lib().mynah_b200_batch_run(self.h, bh, decoder), "batch_run")

    def batch_fetch(self, bh, B):
        tk, fr, nt = (C.c_void_p * B)(), (C.c_void_p * B)(), (C.c_int * B)()
        _check(lib().mynah_b200_batch_fetch(self.h, bh, tk, fr, nt), "batch_fetch")
        return [(_take_i32(tk[b], nt[b]), _take_i32(fr[b], nt[b])) for b in range(B)]

    def batch_free(self, bh):
        lib().mynah_b200_batch_free(bh)
