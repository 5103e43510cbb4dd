"""CPU oracle for the mynah-asr hot path — TEST INFRASTRUCTURE ONLY.

A numpy restatement of the reference's algorithms for the quantised matmul,
the FastConformer encoder, the dw-striding subsampling, the log-mel front end
and the greedy CTC / RNNT / TDT decoders. Nothing in the product imports this
module: it exists so that the CUDA path can be checked against the reference's
arithmetic on machines where the reference sources are absent.

Parity pin: every function here is checked (tests/test_oracle_pin.py) against
  * the ggml block-decode known-answer vectors the reference ships
    (third_party/ingot/tests/fixtures/{Q8_0,Q4_0,Q4_K,Q6_K}.{bin,ref}), and
  * outputs of the reference itself, compiled unmodified into
    oracle/_ref/libmynah_ref.so, committed as fixtures under tests/golden/.

Each function cites the reference file:line it follows (paths relative to the
reference project root). Float work is done in float32 with float64 where the
reference uses double; integer work is exact.
"""
from __future__ import annotations

import numpy as np

f32 = np.float32

# --------------------------------------------------------------------------
# ggml block formats (third_party/ingot/src/dequant.c)
# --------------------------------------------------------------------------
GGML_F32, GGML_F16, GGML_Q4_0, GGML_Q8_0, GGML_Q4_K, GGML_Q6_K = 0, 1, 2, 8, 12, 14
BLOCK_GEOM = {GGML_Q4_0: (32, 18), GGML_Q8_0: (32, 34), GGML_Q4_K: (256, 144), GGML_Q6_K: (256, 210)}


def _f16(b: np.ndarray) -> np.ndarray:
    """little-endian byte pairs [..., 2] -> float32"""
    return np.ascontiguousarray(b).view("<f2").astype(f32)[..., 0]


def dequant_q8_0(raw: np.ndarray) -> np.ndarray:
    """34-byte blocks: f16 d + 32 int8; w = d*q (dequant.c:131-156)."""
    blk = raw.reshape(-1, 34)
    d = _f16(blk[:, 0:2])
    q = blk[:, 2:].view(np.int8).astype(f32)
    return (d[:, None] * q).reshape(-1)


def dequant_q4_0(raw: np.ndarray) -> np.ndarray:
    """18-byte blocks: f16 d + 16 bytes; byte i holds element i (low nibble) and
    element i+16 (high nibble); w = d*(nib-8) (dequant.c:72-83)."""
    blk = raw.reshape(-1, 18)
    d = _f16(blk[:, 0:2])
    q = blk[:, 2:]
    lo = (q & 0x0F).astype(np.int32) - 8
    hi = (q >> 4).astype(np.int32) - 8
    w = np.concatenate([lo, hi], axis=1).astype(f32)
    return (d[:, None] * w).reshape(-1)


def _k4_scale_min(sc: np.ndarray):
    """6-bit packed scales/mins of Q4_K (dequant.c:55-68). sc [nb,12] uint8 ->
    (scale [nb,8], min [nb,8])."""
    s = np.zeros(sc.shape[:-1] + (8,), np.uint8)
    m = np.zeros_like(s)
    s[:, 0:4] = sc[:, 0:4] & 63
    m[:, 0:4] = sc[:, 4:8] & 63
    s[:, 4:8] = (sc[:, 8:12] & 0x0F) | ((sc[:, 0:4] >> 6) << 4)
    m[:, 4:8] = (sc[:, 8:12] >> 4) | ((sc[:, 4:8] >> 6) << 4)
    return s, m


def dequant_q4_k(raw: np.ndarray) -> np.ndarray:
    """144-byte super-blocks of 256: f16 d, f16 dmin, 12 bytes of 6-bit
    scales/mins, 128 bytes of nibbles; eight sub-blocks of 32,
    w = (d*sc)*q - (dmin*m) (dequant.c:222-273)."""
    blk = raw.reshape(-1, 144)
    d = _f16(blk[:, 0:2])
    dmin = _f16(blk[:, 2:4])
    sc, mn = _k4_scale_min(blk[:, 4:16])
    q = blk[:, 16:].reshape(-1, 4, 32)          # four groups of 64 elements
    lo = (q & 0x0F).astype(f32)                  # sub-block 2g
    hi = (q >> 4).astype(f32)                    # sub-block 2g+1
    qq = np.stack([lo, hi], axis=2).reshape(-1, 8, 32)
    dd = (d[:, None] * sc.astype(f32)).astype(f32)
    mm = (dmin[:, None] * mn.astype(f32)).astype(f32)
    return (dd[:, :, None] * qq - mm[:, :, None]).astype(f32).reshape(-1)


def dequant_q6_k(raw: np.ndarray) -> np.ndarray:
    """210-byte super-blocks of 256: ql[128], qh[64], 16 int8 scales, f16 d;
    w = d*sc*(q-32), two halves of 128 (dequant.c:352-445)."""
    blk = raw.reshape(-1, 210)
    nb = blk.shape[0]
    ql = blk[:, 0:128].reshape(nb, 2, 64)
    qh = blk[:, 128:192].reshape(nb, 2, 32)
    sc = blk[:, 192:208].view(np.int8).reshape(nb, 2, 8).astype(f32)
    d = _f16(blk[:, 208:210])
    out = np.zeros((nb, 2, 128), f32)
    l0, l1 = ql[:, :, 0:32], ql[:, :, 32:64]
    q1 = ((l0 & 0x0F) | (((qh >> 0) & 3) << 4)).astype(np.int32) - 32
    q2 = ((l1 & 0x0F) | (((qh >> 2) & 3) << 4)).astype(np.int32) - 32
    q3 = ((l0 >> 4) | (((qh >> 4) & 3) << 4)).astype(np.int32) - 32
    q4 = ((l1 >> 4) | (((qh >> 6) & 3) << 4)).astype(np.int32) - 32
    isx = np.arange(32) // 16
    for j, q in enumerate((q1, q2, q3, q4)):
        s = sc[:, :, isx + 2 * j]               # [nb,2,32]
        out[:, :, 32 * j:32 * j + 32] = ((d[:, None, None] * s).astype(f32) * q.astype(f32))
    return out.reshape(-1)


def ggml_dequant(ggml_type: int, raw: np.ndarray) -> np.ndarray:
    raw = np.ascontiguousarray(raw, dtype=np.uint8).reshape(-1)
    if ggml_type == GGML_F32:
        return raw.view(f32).copy()
    return {GGML_Q8_0: dequant_q8_0, GGML_Q4_0: dequant_q4_0,
            GGML_Q4_K: dequant_q4_k, GGML_Q6_K: dequant_q6_k}[ggml_type](raw)


# --------------------------------------------------------------------------
# mynah-native int8 / int4 (src/qmat.c)
# --------------------------------------------------------------------------
def _round_half_away(v: np.ndarray) -> np.ndarray:
    """(int)(v >= 0 ? v + 0.5f : v - 0.5f) in float32 (qmat.c:33,57,196)."""
    v = v.astype(f32)
    return np.where(v >= 0, (v + f32(0.5)).astype(f32), (v - f32(0.5)).astype(f32)).astype(np.int32)


def quantize_int8(w: np.ndarray):
    """Per-row symmetric int8, scale = amax/127 (qmat.c:19-36)."""
    w = w.astype(f32)
    amax = np.abs(w).max(axis=1)
    scale = np.where(amax > 0, amax / f32(127.0), f32(1.0)).astype(f32)
    inv = (f32(1.0) / scale).astype(f32)
    q = _round_half_away(w * inv[:, None]).astype(np.int8)
    return q, scale


def quantize_int4(w: np.ndarray):
    """Per-group-of-32 symmetric int4: byte j of a group = element 2j | (2j+1)<<4,
    stored value = q+8, scale = amax/7 (qmat.c:38-67)."""
    w = w.astype(f32)
    n, k = w.shape
    g = w.reshape(n, k // 32, 32)
    amax = np.abs(g).max(axis=2)
    scale = np.where(amax > 0, amax / f32(7.0), f32(1.0)).astype(f32)
    inv = (f32(1.0) / scale).astype(f32)
    q = np.clip(_round_half_away(g * inv[:, :, None]), -8, 7)
    packed = ((q[:, :, 0::2] + 8) | ((q[:, :, 1::2] + 8) << 4)).astype(np.uint8)
    return packed.reshape(n, k // 2), scale


def dequant_int8(q: np.ndarray, scale: np.ndarray) -> np.ndarray:
    return q.astype(f32) * scale[:, None].astype(f32)          # qmat.c:153-156


def unpack_int4(q4: np.ndarray) -> np.ndarray:
    """[n,k/2] packed -> [n,k] signed ints in [-8,7] (qmat.c:160-166)."""
    n = q4.shape[0]
    lo = (q4 & 0x0F).astype(np.int32) - 8
    hi = (q4 >> 4).astype(np.int32) - 8
    return np.stack([lo, hi], axis=2).reshape(n, -1)


def dequant_int4(q4: np.ndarray, scale: np.ndarray) -> np.ndarray:
    w = unpack_int4(q4).astype(f32)
    n, k = w.shape
    return (w.reshape(n, k // 32, 32) * scale[:, :, None].astype(f32)).reshape(n, k)


def quantize_act_int8(x: np.ndarray):
    """Per-row absmax activation quantisation: inv = 127/amax, round half away,
    clamp to +-127, returns (qx int8 [T,k], sx = amax/127) (qmat.c:186-202)."""
    x = x.astype(f32)
    amax = np.abs(x).max(axis=1)
    inv = np.where(amax > 0, f32(127.0) / np.where(amax > 0, amax, 1).astype(f32), f32(0)).astype(f32)
    q = np.clip(_round_half_away(x * inv[:, None]), -127, 127).astype(np.int8)
    sx = np.where(amax > 0, amax / f32(127.0), f32(0)).astype(f32)
    return q, sx


def int_dots_q8(qx: np.ndarray, qw: np.ndarray) -> np.ndarray:
    """Exact int32 row dots [T,n] (qmat.c:285-300: one int32 per (t, row))."""
    return qx.astype(np.int32) @ qw.astype(np.int32).T


def int_dots_q4(qx: np.ndarray, qw_signed: np.ndarray) -> np.ndarray:
    """Exact per-group int32 dots [T,n,k/32] (qmat.c:347-362)."""
    T, k = qx.shape
    n = qw_signed.shape[0]
    a = qx.astype(np.int32).reshape(T, 1, k // 32, 32)
    b = qw_signed.astype(np.int32).reshape(1, n, k // 32, 32)
    return (a * b).sum(axis=3)


def qmat_mul_a8_q8(x, q, scale):
    """int8 activations x int8 weights: (float)int32 * ws * sx (qmat.c:299)."""
    qx, sx = quantize_act_int8(x)
    dots = int_dots_q8(qx, q).astype(f32)
    return ((dots * scale[None, :].astype(f32)).astype(f32) * sx[:, None]).astype(f32)


def qmat_mul_a8_q4(x, q4, scale):
    """Per group: acc += (float)int32_g * scale_g, groups in ascending order,
    then * sx (qmat.c:347-363)."""
    qx, sx = quantize_act_int8(x)
    dots = int_dots_q4(qx, unpack_int4(q4)).astype(f32)         # [T,n,G]
    acc = np.zeros(dots.shape[:2], f32)
    for g in range(dots.shape[2]):
        acc = (acc + (dots[:, :, g] * scale[None, :, g].astype(f32)).astype(f32)).astype(f32)
    return (acc * sx[:, None]).astype(f32)


def gemm_wt(x, w):
    """out[T,n] = x[T,k] @ W[n,k]^T in float32 (backend.c:68-81)."""
    return (x.astype(f32) @ w.astype(f32).T).astype(f32)


# --------------------------------------------------------------------------
# activations (src/qmat.h:31-35, src/backend.c:88-108)
# --------------------------------------------------------------------------
def sigmoid(x):
    x = x.astype(f32)
    e = np.exp(-np.abs(x)).astype(f32)
    return np.where(x >= 0, f32(1) / (f32(1) + e), e / (f32(1) + e)).astype(f32)


def silu(x):
    return (x.astype(f32) * sigmoid(x)).astype(f32)


# --------------------------------------------------------------------------
# log-mel front end (src/features.c:106-167)
# --------------------------------------------------------------------------
def log_mel(audio, mel_fb, window, n_fft=512, hop=160, preemph=0.97, guard=2.0 ** -24,
            normalize_per_feature=False):
    """audio float32 [S] -> (feats [T, n_mels] float32, valid). T = 1 + S//hop,
    rows >= valid = S//hop stay zero. Double precision inside, like the reference."""
    audio = np.asarray(audio, f32)
    S = audio.shape[0]
    n_mels = mel_fb.shape[1]
    pad = n_fft // 2
    T, valid = 1 + S // hop, S // hop
    y = np.zeros(S + 2 * pad, np.float64)
    if S > 0:
        y[pad] = audio[0]
        y[pad + 1:pad + S] = audio[1:].astype(np.float64) - preemph * audio[:-1].astype(np.float64)
    win = np.zeros(n_fft, np.float64)
    off = (n_fft - window.shape[0]) // 2
    win[off:off + window.shape[0]] = window.astype(np.float64)
    feats = np.zeros((T, n_mels), f32)
    if valid > 0:
        idx = np.arange(valid)[:, None] * hop + np.arange(n_fft)[None, :]
        spec = np.fft.rfft(y[idx] * win[None, :], axis=1)
        power = spec.real ** 2 + spec.imag ** 2
        acc = power @ mel_fb.astype(np.float64)
        feats[:valid] = np.log(acc + guard).astype(f32)
    if normalize_per_feature and valid > 1:
        v = feats[:valid].astype(np.float64)
        mu = v.mean(axis=0)
        var = ((v - mu) ** 2).sum(axis=0) / (valid - 1)
        feats[:valid] = ((v - mu) / (np.sqrt(var) + 1e-5)).astype(f32)
    return feats, valid


# --------------------------------------------------------------------------
# dw-striding subsampling (src/subsampling.c:107-269)
# --------------------------------------------------------------------------
def _conv3x3_s2(x, w, b, pl_t, pr_t, pl_f, pr_f, depthwise):
    """x [C_in,T,F] -> [C_out,To,Fo]; kernel 3, stride 2, zero padding."""
    C_in, T, F = x.shape
    xp = np.zeros((C_in, T + pl_t + pr_t, F + pl_f + pr_f), f32)
    xp[:, pl_t:pl_t + T, pl_f:pl_f + F] = x
    To = (xp.shape[1] - 3) // 2 + 1
    Fo = (xp.shape[2] - 3) // 2 + 1
    C_out = w.shape[0]
    out = np.zeros((C_out, To, Fo), f32)
    for dt in range(3):
        for df in range(3):
            patch = xp[:, dt:dt + 2 * To:2, df:df + 2 * Fo:2][:, :To, :Fo]
            if depthwise:
                out += w[:, 0, dt, df][:, None, None] * patch
            else:
                out += np.einsum("oc,ctf->otf", w[:, :, dt, df], patch).astype(f32)
    return (out + b[:, None, None]).astype(f32)


def subsampling_forward(W, feats, causal=False):
    """feats [T,n_mels] -> [T', d_model]. W: dict with conv_in_w/b, dw_w/b[2],
    pw_w/b[2], lin_w/b (names as src/subsampling.h:13-17)."""
    pl, pr = (2, 1) if causal else (1, 1)
    a = _conv3x3_s2(feats[None].astype(f32), W["conv_in_w"], W["conv_in_b"], pl, pr, pl, pr, False)
    a = np.maximum(a, 0)
    for i in range(2):
        bq = _conv3x3_s2(a, W["dw_w"][i], W["dw_b"][i], pl, pr, pl, pr, True)
        C, To, Fo = bq.shape
        pw = W["pw_w"][i].reshape(C, C)
        a = (pw @ bq.reshape(C, -1)).astype(f32).reshape(C, To, Fo) + W["pw_b"][i][:, None, None]
        a = np.maximum(a, 0).astype(f32)
    C, To, Fo = a.shape
    flat = a.transpose(1, 0, 2).reshape(To, C * Fo)            # channel-major flatten
    return (gemm_wt(flat, W["lin_w"]) + W["lin_b"][None, :]).astype(f32)


# --------------------------------------------------------------------------
# encoder (src/encoder.c)
# --------------------------------------------------------------------------
def layer_norm(x, w, b, eps=1e-5):
    """Mean/var in double, ((x-mu)*inv)*w + b in float (encoder.c:25-37)."""
    xd = x.astype(np.float64)
    mu = xd.mean(axis=1, keepdims=True)
    var = ((xd - mu) ** 2).mean(axis=1, keepdims=True)
    inv = (1.0 / np.sqrt(var + eps)).astype(f32)
    return (((x.astype(f32) - mu.astype(f32)) * inv).astype(f32) * w + b).astype(f32)


def pos_emb(T, d):
    """[2T-1, d], positions T-1 .. -(T-1), sin/cos interleaved (encoder.c:201-211)."""
    pos = (T - 1 - np.arange(2 * T - 1, dtype=np.float64))[:, None]
    j = np.arange(d // 2, dtype=np.float64)[None, :]
    freq = pos * np.power(10000.0, -2.0 * j / d)
    pe = np.zeros((2 * T - 1, d), f32)
    pe[:, 0::2] = np.sin(freq).astype(f32)
    pe[:, 1::2] = np.cos(freq).astype(f32)
    return pe


def _lin(L, name, x):
    """A quantisable linear; L[name] is the EFFECTIVE f32 weight (what the
    reference holds after its eager block decode, src/weights.c:90-115)."""
    if L.get("a8") and (name + "_q8") in L:
        # int8 activations x reference-native int8 weights for every row count: the reference's arithmetic below
        # 17 rows, and above with MYNAH_ASR_QGEMM=1 (src/qmat.c:508-551, 598-643)
        q, s = L[name + "_q8"]
        y = qmat_mul_a8_q8(x, q, s)
    else:
        y = gemm_wt(x, L[name])
    b = L.get(name + "_b")
    return y if b is None else (y + b[None, :]).astype(f32)


def attention(L, x, pe, H, left=-1, right=-1):
    """Rel-pos MHSA with bias_u/bias_v and the closed-form rel-shift
    bd[t, T-1+j-t]; softmax over the chunked-limited window when left >= 0
    (encoder.c:315-410, windows :371-381)."""
    T, d = x.shape
    dk = d // H
    scaling = f32(1.0) / np.sqrt(f32(dk))
    q, k, v = _lin(L, "q_w", x), _lin(L, "k_w", x), _lin(L, "v_w", x)
    rk = gemm_wt(pe, L["relk_w"])                               # [2T-1, d]
    chunk = right + 1 if left >= 0 else 1
    lc = left // chunk if left >= 0 else 0
    t_idx = np.arange(T)
    ctx = np.zeros((T, d), f32)
    rel = (T - 1) + t_idx[None, :] - t_idx[:, None]             # [t, j] -> p
    for h in range(H):
        sl = slice(h * dk, (h + 1) * dk)
        ac = ((q[:, sl] + L["bias_u"][h]) @ k[:, sl].T).astype(f32)
        bd = ((q[:, sl] + L["bias_v"][h]) @ rk[:, sl].T).astype(f32)
        s = ((ac + np.take_along_axis(bd, rel, axis=1)) * scaling).astype(f32)
        if left >= 0:
            tc = t_idx // chunk
            j0 = np.maximum((tc - lc) * chunk, 0)
            j1 = np.minimum((tc + 1) * chunk, T)
            mask = (t_idx[None, :] >= j0[:, None]) & (t_idx[None, :] < j1[:, None])
            s = np.where(mask, s, f32(-3.0e38))
        else:
            mask = None
        m = s.max(axis=1, keepdims=True)
        e = np.exp((s - m).astype(f32)).astype(f32)
        if mask is not None:
            e = np.where(mask, e, f32(0))
        p = (e * (f32(1.0) / e.sum(axis=1, keepdims=True, dtype=f32))).astype(f32)
        ctx[:, sl] = (p @ v[:, sl]).astype(f32)
    return _lin(L, "o_w", ctx)


def conv_module(L, x, causal):
    """pw1 -> GLU -> depthwise k -> folded BN affine or LN -> SiLU -> pw2
    (encoder.c:413-460)."""
    T, d = x.shape
    h2 = _lin(L, "pw1_w", x)
    g = (h2[:, :d] * sigmoid(h2[:, d:])).astype(f32)
    dw = L["dw_w"].reshape(d, -1)
    k = dw.shape[1]
    pc = k - 1 if causal else (k - 1) // 2
    gp = np.zeros((T + k - 1, d), f32)
    gp[pc:pc + T] = g
    c = np.zeros((T, d), f32)
    if L.get("dw_b") is not None:
        c += L["dw_b"][None, :]
    for j in range(k):
        c = (c + dw[None, :, j] * gp[j:j + T]).astype(f32)
    if L.get("cnorm_scale") is not None:
        g2 = (c * L["cnorm_scale"][None, :] + L["cnorm_shift"][None, :]).astype(f32)
    else:
        g2 = layer_norm(c, L["cnorm_w"], L["cnorm_b"])
    return _lin(L, "pw2_w", silu(g2))


def half_ffn(L, x, which):
    """LN -> linear1 (+b) -> SiLU -> linear2 (+b) (encoder.c:464-482)."""
    p = "ff2" if which else "ff1"
    h = layer_norm(x, L["ln_" + p + "_w"], L["ln_" + p + "_b"])
    return _lin(L, p + "_w2", silu(_lin(L, p + "_w1", h)))


def encoder_layer(L, x, pe, H, causal, left=-1, right=-1):
    """Macaron block, residual weights 0.5/1/1/0.5, output LN (encoder.c:485-519)."""
    x = (x + f32(0.5) * half_ffn(L, x, 0)).astype(f32)
    x = (x + attention(L, layer_norm(x, L["ln_att_w"], L["ln_att_b"]), pe, H, left, right)).astype(f32)
    x = (x + conv_module(L, layer_norm(x, L["ln_conv_w"], L["ln_conv_b"]), causal)).astype(f32)
    x = (x + f32(0.5) * half_ffn(L, x, 1)).astype(f32)
    return layer_norm(x, L["ln_out_w"], L["ln_out_b"])


def encoder_post(M, x, prompt_id=0):
    """encoder_projector when present, else identity (encoder.c:573-590); for a
    prompt-conditioned model the one-hot prompt is concatenated to every frame and goes
    through linear_1 (+b, ReLU) and linear_2 (+b) first (encoder.c:591-614)."""
    if M.get("encproj_w") is None:
        return x.copy()
    if M.get("prompt_l1_w") is not None:
        T, d = x.shape
        np_ = M["prompt_l1_w"].shape[1] - d
        cat = np.zeros((T, d + np_), f32)
        cat[:, :d] = x
        cat[:, d + prompt_id] = 1.0
        mid = np.maximum(gemm_wt(cat, M["prompt_l1_w"]) + M["prompt_l1_b"][None, :], f32(0)).astype(f32)
        x = (gemm_wt(mid, M["prompt_l2_w"]) + M["prompt_l2_b"][None, :]).astype(f32)
    return (gemm_wt(x, M["encproj_w"]) + M["encproj_b"][None, :]).astype(f32)


def encoder_forward(M, feats, left=-1, right=-1, raw=False, n_layers=None, prompt_id=0):
    """feats [T_mel, n_mels] (valid frames) -> [T, d_out] (encoder.c:1013-1039)."""
    x = subsampling_forward(M["ss"], feats, M["causal"])
    if M.get("xscale", 1.0) != 1.0:
        x = (x * f32(M["xscale"])).astype(f32)
    T, d = x.shape
    pe = pos_emb(T, d)
    for L in M["layers"][:n_layers]:
        x = encoder_layer(L, x, pe, M["n_heads"], M["causal"], left, right)
    return x if raw else encoder_post(M, x, prompt_id)


# --------------------------------------------------------------------------
# decoders (src/decoder_ctc.c, src/decoder.c)
# --------------------------------------------------------------------------
def _argmax_bias(lg, bias):
    """First index of the maximum of logits+bias (decoder.c:113-121)."""
    return int(np.argmax((lg + bias).astype(f32)))


def ctc_decode(enc, w, b):
    """argmax(logit+b), collapse repeats, drop blank = V-1, first frame per token
    (decoder_ctc.c:36-61)."""
    logits = gemm_wt(enc, w)
    best = np.argmax((logits + b[None, :]).astype(f32), axis=1)
    blank = w.shape[0] - 1
    toks, frames, prev = [], [], -1
    for t, k in enumerate(best):
        if k != prev and k != blank:
            toks.append(int(k)); frames.append(t)
        prev = k
    return toks, frames


def _lstm_pred_step(D, state, token):
    """Stacked LSTM step + decoder_projector, gates i,f,g,o (decoder.c:73-99)."""
    H = D["hidden"]
    x = D["embedding"][token]
    for l in range(D["n_layers"]):
        z = (D["b_ih"][l] + D["b_hh"][l]).astype(f32)
        z = (z + D["w_ih"][l] @ x).astype(f32)
        z = (z + D["w_hh"][l] @ state["h"][l]).astype(f32)
        ig, fg = sigmoid(z[:H]), sigmoid(z[H:2 * H])
        gg, og = np.tanh(z[2 * H:3 * H]).astype(f32), sigmoid(z[3 * H:])
        state["c"][l] = (fg * state["c"][l] + ig * gg).astype(f32)
        state["h"][l] = (og * np.tanh(state["c"][l]).astype(f32)).astype(f32)
        x = state["h"][l]
    state["g"] = (D["proj_b"] + D["proj_w"] @ state["h"][D["n_layers"] - 1]).astype(f32)


def greedy_decode(D, enc):
    """RNNT (durations empty) or TDT greedy from a fresh state; SOS = blank.
    RNNT: per frame emit until blank or max_symbols (decoder.c:183-265; the
    blocked blank-run batching there is an optimisation with identical
    semantics). TDT: t += duration with the blank/max_symbols rules
    (decoder.c:129-181). Returns (tokens, frames)."""
    H = D["hidden"]
    st = {"h": [np.zeros(H, f32) for _ in range(D["n_layers"])],
          "c": [np.zeros(H, f32) for _ in range(D["n_layers"])], "g": None}
    _lstm_pred_step(D, st, D["blank"])
    T = enc.shape[0]
    V = D["vocab"]
    durs = D.get("durations") or []
    toks, frames = [], []
    t = 0
    if durs:
        emitted_here = 0
        while t < T:
            joint = np.maximum(enc[t] + st["g"], 0).astype(f32)
            logits = (D["head_w"] @ joint).astype(f32)
            k = _argmax_bias(logits[:V], D["head_b"][:V])
            dur = durs[_argmax_bias(logits[V:], D["head_b"][V:])]
            if k != D["blank"]:
                toks.append(k); frames.append(t)
                _lstm_pred_step(D, st, k)
                emitted_here += 1
                if dur == 0 and emitted_here >= D["max_symbols"]:
                    dur = 1
            elif dur == 0:
                dur = 1
            if dur > 0:
                emitted_here = 0
            t += dur
        return toks, frames
    while t < T:
        for _ in range(D["max_symbols"]):
            joint = np.maximum(enc[t] + st["g"], 0).astype(f32)
            k = _argmax_bias((D["head_w"] @ joint).astype(f32), D["head_b"])
            if k == D["blank"]:
                break
            toks.append(k); frames.append(t)
            _lstm_pred_step(D, st, k)
        t += 1
    return toks, frames


# ------------------------------------------------------------------ AED decoder
def _aed_ln(x, w, b):
    """ln of src/decoder_aed.c:24-31: mean / variance in double, eps 1e-5."""
    x64 = x.astype(np.float64)
    mu = x64.mean()
    var = ((x64 - mu) ** 2).mean()
    inv = np.float32(1.0 / np.sqrt(var + 1e-5))
    return ((x64 - mu) * inv).astype(np.float32) * w + b


def _aed_attend(q, K, V, H):
    """attend of src/decoder_aed.c:117-131: one query over n_kv keys, per head,
    scores scaled by 1/sqrt(dk), f32 softmax."""
    d = q.shape[0]
    dk = d // H
    out = np.empty(d, np.float32)
    scale = np.float32(1.0 / np.sqrt(np.float32(dk)))
    for h in range(H):
        sl = slice(h * dk, (h + 1) * dk)
        sc = (K[:, sl] @ q[sl]).astype(np.float32) * scale
        e = np.exp(sc - sc.max(), dtype=np.float32)
        pr = e * np.float32(1.0 / e.sum(dtype=np.float32))
        out[sl] = pr @ V[:, sl]
    return out


def aed_decode(A, enc, prompt, eos, cap):
    """mynah_asr_aed_decode (src/decoder_aed.c:139-232): greedy autoregressive decode of the
    pre-LN transformer decoder; returns the generated tokens (prompt and EOS excluded).
    A: dict with emb, pos, embln_w/b, fin_w/b, head_w/b, optional proj_w/b, n_heads, max_seq and
    layers[...] of ln_{self,cross,ffn}_w/b, s{q,k,v,o}_w/b, c{q,k,v,o}_w/b, ff1_w/b, ff2_w/b."""
    H = A["n_heads"]
    prompt = list(prompt)
    if not prompt:
        return None
    max_len = min(len(prompt) + cap, A["max_seq"])                      # :144-146
    encp = gemm_wt(enc, A["proj_w"]) + A["proj_b"] if A.get("proj_w") is not None else enc     # :149-157
    cross = [(gemm_wt(encp, L["ck_w"]) + L["ck_b"], gemm_wt(encp, L["cv_w"]) + L["cv_b"]) for L in A["layers"]]   # :171-178
    d = A["emb"].shape[1]
    SK = [np.zeros((max_len, d), np.float32) for _ in A["layers"]]
    SV = [np.zeros((max_len, d), np.float32) for _ in A["layers"]]
    out, cur = [], prompt[0]
    for p in range(max_len):
        x = _aed_ln(A["emb"][cur] + A["pos"][p], A["embln_w"], A["embln_b"])      # :183-185
        for li, L in enumerate(A["layers"]):
            xn = _aed_ln(x, L["ln_self_w"], L["ln_self_b"])
            q = gemm_wt(xn[None], L["sq_w"])[0] + L["sq_b"]
            SK[li][p] = gemm_wt(xn[None], L["sk_w"])[0] + L["sk_b"]
            SV[li][p] = gemm_wt(xn[None], L["sv_w"])[0] + L["sv_b"]
            att = _aed_attend(q, SK[li][:p + 1], SV[li][:p + 1], H)             # causal: keys 0..p
            x = x + (gemm_wt(att[None], L["so_w"])[0] + L["so_b"])
            xn = _aed_ln(x, L["ln_cross_w"], L["ln_cross_b"])
            q = gemm_wt(xn[None], L["cq_w"])[0] + L["cq_b"]
            att = _aed_attend(q, cross[li][0], cross[li][1], H)
            x = x + (gemm_wt(att[None], L["co_w"])[0] + L["co_b"])
            xn = _aed_ln(x, L["ln_ffn_w"], L["ln_ffn_b"])
            ff = np.maximum(gemm_wt(xn[None], L["ff1_w"])[0] + L["ff1_b"], np.float32(0.0))
            x = x + (gemm_wt(ff[None], L["ff2_w"])[0] + L["ff2_b"])
        if p + 1 < len(prompt):                                                  # :211-214
            cur = prompt[p + 1]
            continue
        logits = gemm_wt(_aed_ln(x, A["fin_w"], A["fin_b"])[None], A["head_w"])[0] + A["head_b"]
        best = int(np.argmax(logits))                                            # first maximum, as :217-218
        if best == eos or len(out) >= cap:
            break
        out.append(best)
        cur = best
    return np.asarray(out, np.int32)


# ------------------------------------------------------------------ CTC forced alignment (src/align.c)
ALIGN_NEG_BIG, ALIGN_UNREACHABLE = f32(-1.0e30), f32(-1.0e29)


def align_min_frames(tokens):
    """One frame per token plus a blank between identical neighbours (align.c:24-30)."""
    return len(tokens) + sum(1 for a, b in zip(tokens[1:], tokens[:-1]) if a == b)


def align_ctc(scores, tokens, blank):
    """Viterbi over blank, tok0, blank, tok1, ..., blank (align.c:32-97): moves stay / from s-1 / from s-2 (only into a
    label that differs from the label two states back), the later candidate wins only when strictly greater, states
    that can no longer finish or cannot be reached yet are pruned, raw logits as scores. Returns (rc, t0, t1): first
    and last frame of every token's run, rc -1 when the arguments are bad or no path exists."""
    scores = np.asarray(scores, f32)
    T, V = scores.shape
    n = len(tokens)
    if T <= 0 or V <= 0 or n <= 0 or blank < 0 or blank >= V or any(t < 0 or t >= V or t == blank for t in tokens):
        return -1, [], []
    if T < align_min_frames(tokens):
        return -1, [], []
    S = 2 * n + 1
    ext = np.full(S, blank, np.int64)
    ext[1::2] = tokens
    can_skip = np.zeros(S, bool)
    can_skip[2:] = (ext[2:] != blank) & (ext[2:] != ext[:-2])
    prv = np.full(S, ALIGN_NEG_BIG, f32)
    prv[0], prv[1] = scores[0, ext[0]], scores[0, ext[1]]
    bp = np.zeros((T, S), np.uint8)
    for t in range(1, T):
        s_lo, s_hi = max(S - 2 * (T - t), 0), min(2 * t + 1, S - 1)
        best, frm = prv.copy(), np.zeros(S, np.uint8)
        m1 = np.zeros(S, bool); m1[1:] = prv[:-1] > best[1:]
        best[m1] = np.concatenate([[ALIGN_NEG_BIG], prv[:-1]])[m1]; frm[m1] = 1
        m2 = np.zeros(S, bool); m2[2:] = can_skip[2:] & (prv[:-2] > best[2:])
        best[m2] = np.concatenate([[ALIGN_NEG_BIG, ALIGN_NEG_BIG], prv[:-2]])[m2]; frm[m2] = 2
        cur = np.where(best > ALIGN_UNREACHABLE, (best + scores[t, ext]).astype(f32), ALIGN_NEG_BIG).astype(f32)
        live = np.zeros(S, bool); live[s_lo:s_hi + 1] = True
        cur[~live] = ALIGN_NEG_BIG; frm[~live] = 0
        bp[t], prv = frm, cur
    s = S - 1 if prv[S - 1] >= prv[S - 2] else S - 2
    if prv[s] <= ALIGN_UNREACHABLE:
        return -1, [], []
    t0, t1 = [-1] * n, [-1] * n
    for t in range(T - 1, -1, -1):
        if s % 2 == 1:
            j = s // 2
            if t1[j] < 0:
                t1[j] = t
            t0[j] = t
        s -= int(bp[t, s])
    return (0 if all(v >= 0 for v in t0) else -1), t0, t1


# ------------------------------------------------------------------ voice activity (src/vad.c) and segment planning
class Vad:
    """mynah_asr_vad (src/vad.c): cfg = the "vad" section of mynah.json, W = {tensor name: f32 array}. One frame of
    frame_samples in, one speech probability out, with the LSTM state and the lookbehind carried between calls."""

    def __init__(self, cfg, W):
        self.c, self.W = cfg, W
        self.reset()

    def reset(self):
        H = self.c["lstm_hidden"]
        self.look = np.zeros(self.c["context_samples"], f32)
        self.h, self.cell = np.zeros(H, f32), np.zeros(H, f32)

    def features(self, samples):
        """lookbehind | frame (zero-padded) | reflect pad -> STFT magnitude -> conv blocks (vad.c:316-352): [hidden]"""
        c = self.c
        C, F, P = c["context_samples"], c["frame_samples"], c["reflect_pad"]
        buf = np.zeros(C + F + P, f32)
        buf[:C] = self.look
        buf[C:C + len(samples)] = samples
        N = C + F
        buf[N:] = buf[N - 2 - np.arange(P)]
        self.look = buf[N - C:N].copy()
        T0, nf, hop, B = c["stft_frames"], c["n_fft"], c["hop_length"], c["n_bins"]
        win = np.stack([buf[f * hop:f * hop + nf] for f in range(T0)])
        spec = gemm_wt(self.W["stft.forward_basis_buffer"].reshape(2 * B, nf), win)       # [2B, T0]
        x = np.sqrt((spec[:B] * spec[:B] + spec[B:] * spec[B:]).astype(f32)).astype(f32)
        for i, (st, (pl, pr)) in enumerate(zip(c["encoder_strides"], c["encoder_pads"])):
            w, b = self.W[f"encoder.{i}.reparam_conv.weight"], self.W[f"encoder.{i}.reparam_conv.bias"]
            cout, cin, k = w.shape
            t_in = x.shape[1]
            t_out = (t_in + pl + pr - k) // st + 1
            xp = np.zeros((cin, t_in + pl + pr), f32)
            xp[:, pl:pl + t_in] = x
            col = np.stack([xp[:, t * st:t * st + k].reshape(-1) for t in range(t_out)])   # [t_out, cin * k]
            x = np.maximum(gemm_wt(w.reshape(cout, cin * k), col) + b[:, None], f32(0)).astype(f32)
        return x[:, 0]

    def feed(self, samples):
        """mynah_asr_vad_feed (vad.c:316-385)."""
        H = self.c["lstm_hidden"]
        x = self.features(np.asarray(samples, f32))
        z = (self.W["decoder.rnn.bias_ih"] + self.W["decoder.rnn.bias_hh"]).astype(f32)
        z = (z + self.W["decoder.rnn.weight_ih"] @ x).astype(f32)
        z = (z + self.W["decoder.rnn.weight_hh"] @ self.h).astype(f32)
        ig, fg, gg, og = sigmoid(z[:H]), sigmoid(z[H:2 * H]), np.tanh(z[2 * H:3 * H]).astype(f32), sigmoid(z[3 * H:])
        self.cell = (fg * self.cell + ig * gg).astype(f32)
        self.h = (og * np.tanh(self.cell).astype(f32)).astype(f32)
        acc = f32(self.W["decoder.decoder.2.bias"][0]) + f32(np.sum(self.W["decoder.decoder.2.weight"].reshape(-1) * np.maximum(self.h, 0), dtype=f32))
        return float(sigmoid(np.array([acc], f32))[0])

    def probs(self, samples):
        self.reset()
        F = self.c["frame_samples"]
        return [self.feed(samples[o:o + F]) for o in range(0, len(samples), F)]


def vad_spans_from_probs(cfg, probs, n_samples, sample_rate=16000):
    """The hysteresis of mynah_asr_vad_seg_feed / _finish and the padding of mynah_asr_vad_pad_spans
    (vad.c:417-474): spans [t0, t1) in samples."""
    F = cfg["frame_samples"]
    ms = lambda v: float(sample_rate) * float(v) / 1000.0
    spans, trig, start, temp_end = [], False, 0, -1
    for i, p in enumerate(probs):
        cur = F * i
        if p >= cfg["threshold"]:
            temp_end = -1
            if not trig:
                trig, start = True, cur
            continue
        if p < cfg["neg_threshold"] and trig:
            if temp_end < 0:
                temp_end = cur
            if float(cur - temp_end) < ms(cfg["min_silence_ms"]):
                continue
            end, trig, temp_end = temp_end, False, -1
            if float(end - start) > ms(cfg["min_speech_ms"]):
                spans.append([start, end])
    if trig and float(n_samples - start) > ms(cfg["min_speech_ms"]):
        spans.append([start, n_samples])
    pad = int(float(sample_rate) * float(cfg["speech_pad_ms"]) / 1000.0)
    for i in range(len(spans)):
        if i == 0:
            spans[0][0] = max(spans[0][0] - pad, 0)
        if i != len(spans) - 1:
            gap = spans[i + 1][0] - spans[i][1]
            if gap < 2 * pad:
                spans[i][1] += gap // 2
                spans[i + 1][0] = max(spans[i + 1][0] - gap // 2, 0)
            else:
                spans[i][1] = min(spans[i][1] + pad, n_samples)
                spans[i + 1][0] = max(spans[i + 1][0] - pad, 0)
        else:
            spans[i][1] = min(spans[i][1] + pad, n_samples)
    return [tuple(s) for s in spans]


def find_split_point(s, lo, hi, sr):
    """Centre of the 20 ms window of least energy in [lo, hi), windows every 10 ms, the first minimum wins; the
    energy is a double sum of squares (src/mynah_asr.c:1178-1192)."""
    win = sr // 50
    hop = win // 2
    best, best_pos = 1e300, hi
    p = lo
    while p + win <= hi:
        v = s[p:p + win].astype(np.float64)
        e = 0.0
        for x in v:                       # the reference's summation order
            e += x * x
        if e < best:
            best, best_pos = e, p + win // 2
        p += hop
    return best_pos


def plan_segments(samples, sr, seg_sec, vad_spans=None, context_sec=0.6):
    """plan_segments / plan_segments_vad (src/mynah_asr.c:1216-1323): [(offset, length)]. vad_spans: padded speech
    spans or None for the energy planner."""
    n = len(samples)
    seg_max = int(seg_sec * sr)

    def cut(cur, stop, bound_end):
        out = []
        while cur < stop:
            end = stop
            if stop - cur > seg_max + seg_max // 10:
                hi = cur + seg_max
                lo = hi - 20 * sr if seg_max > 20 * sr else cur + sr
                if lo <= cur:
                    lo = cur + 1
                end = find_split_point(samples, lo, hi, sr)
                if bound_end and (end <= cur or end > stop):
                    end = hi
            if end <= cur:
                end = cur + 1
            out.append((cur, end - cur))
            cur = end
        return out
    if vad_spans is not None and n > 0:
        ctx = int(context_sec * sr)
        sp = [[max(a - ctx, 0), min(b + ctx, n)] for a, b in vad_spans]
        merged = []
        for a, b in sp:
            if merged and a <= merged[-1][1]:
                merged[-1][1] = max(merged[-1][1], b)
            else:
                merged.append([a, b])
        segs = [s for a, b in merged for s in cut(a, b, True)]
        if segs or len(vad_spans) == 0:
            return segs if segs else [(0, 0)]
    segs = cut(0, n, False)
    return segs if segs else [(0, 0)]


# ------------------------------------------------------------------ cache-aware streaming
class EncStream:
    """State of mynah_asr_enc_stream (src/encoder.h:93-108): per-layer K/V caches of up to `left`
    frames, conv caches of k-1 GLU rows, and the subsampling's one-frame caches."""

    def __init__(self, M, left, right, n_mels):
        self.M, self.left, self.right, self.q = M, left, right, right + 1
        d, nl = M["layers"][0]["q_w"].shape[1], len(M["layers"])
        k = M["layers"][0]["dw_w"].reshape(d, -1).shape[1]
        self.kc = [np.zeros((0, d), f32) for _ in range(nl)]
        self.vc = [np.zeros((0, d), f32) for _ in range(nl)]
        self.cc = [np.zeros((k - 1, d), f32) for _ in range(nl)]
        self.valid = 0
        C = M["ss"]["conv_in_w"].shape[0]
        self.ss_first = True
        F, self.ss_cache = n_mels, []
        for s in range(3):                                   # ss_stream_init (src/subsampling.c:272-285)
            self.ss_cache.append(np.zeros((1 if s == 0 else C, F), f32))
            F = F // 2 + 1

    def need(self):
        """mynah_asr_enc_stream_need (src/encoder.c:685-689)."""
        return 1 + 8 * self.right if (self.valid == 0 and self.ss_first) else 8 * (self.right + 1)


def _ss_stream_stage(x, first, last, cache, w, b, depthwise):
    """stream_stage (src/subsampling.c:289-318): time axis = [zero if first][cached frame][chunk][zero if last],
    valid stride-2 conv in time, (2,1) padding in frequency; the cache becomes the chunk's last frame."""
    C, T, F = x.shape
    lp, rp = (2 if first else 1), (1 if last else 0)
    xp = np.zeros((C, T + lp + rp, F), f32)
    xp[:, lp - 1] = cache
    xp[:, lp:lp + T] = x
    cache[...] = x[:, T - 1]
    return _conv3x3_s2(xp, w, b, 0, 0, 2, 1, depthwise)


def ss_stream_step(W, st, mel, is_last):
    """mynah_asr_ss_stream_step (src/subsampling.c:320-370): mel chunk [n, n_mels] -> [q, d_model]."""
    a = np.maximum(_ss_stream_stage(mel[None].astype(f32), st.ss_first, is_last, st.ss_cache[0], W["conv_in_w"], W["conv_in_b"], False), 0)
    for i in range(2):
        bq = _ss_stream_stage(a, st.ss_first, is_last, st.ss_cache[i + 1], W["dw_w"][i], W["dw_b"][i], True)
        C, To, Fo = bq.shape
        a = (W["pw_w"][i].reshape(C, C) @ bq.reshape(C, -1)).astype(f32).reshape(C, To, Fo) + W["pw_b"][i][:, None, None]
        a = np.maximum(a, 0).astype(f32)
    st.ss_first = False
    C, To, Fo = a.shape
    flat = a.transpose(1, 0, 2).reshape(To, C * Fo)
    return (gemm_wt(flat, W["lin_w"]) + W["lin_b"][None, :]).astype(f32)


def _stream_attention(L, x, kn, vn, pe, H, kc, vc):
    """stream_attention (src/encoder.c:695-760): Q query rows over keys [valid cache ; chunk], no mask,
    rel-shift index p = (K-1) - (valid + t) + j."""
    Q, d = x.shape
    valid = kc.shape[0]
    K = valid + Q
    dk = d // H
    scaling = f32(1.0) / np.sqrt(f32(dk))
    q = _lin(L, "q_w", x)
    kk, vv = np.concatenate([kc, kn]), np.concatenate([vc, vn])
    rk = gemm_wt(pe, L["relk_w"])                             # [2K-1, d]
    ctx = np.zeros((Q, d), f32)
    for h in range(H):
        sl = slice(h * dk, (h + 1) * dk)
        bd = ((q[:, sl] + L["bias_v"][h]) @ rk[:, sl].T).astype(f32)
        ac = ((q[:, sl] + L["bias_u"][h]) @ kk[:, sl].T).astype(f32)
        for t in range(Q):
            base = K - 1 - valid - t
            s = ((ac[t] + bd[t, base:base + K]) * scaling).astype(f32)
            e = np.exp((s - s.max()).astype(f32)).astype(f32)
            pr = (e * (f32(1.0) / e.sum(dtype=f32))).astype(f32)
            ctx[t, sl] = (pr @ vv[:, sl]).astype(f32)
    return _lin(L, "o_w", ctx)


def _stream_conv_module(L, x, cache):
    """stream_conv_module (src/encoder.c:779-807): GLU rows appended to the k-1 cached ones, depthwise
    conv over the k rows ending at each new one, LayerNorm, SiLU, pw2. Returns (out, new cache)."""
    Q, d = x.shape
    h2 = _lin(L, "pw1_w", x)
    g = (h2[:, :d] * sigmoid(h2[:, d:])).astype(f32)
    gp = np.concatenate([cache, g])
    dw = L["dw_w"].reshape(d, -1)
    k = dw.shape[1]
    c = np.zeros((Q, d), f32)
    for j in range(k):
        c = (c + dw[None, :, j] * gp[j:j + Q]).astype(f32)
    return _lin(L, "pw2_w", silu(layer_norm(c, L["cnorm_w"], L["cnorm_b"]))), gp[Q:].copy()


def enc_stream_step(st, mel, is_last=False, prompt_id=0):
    """mynah_asr_enc_stream_step (src/encoder.c:809-872): one chunk of mel frames [n, n_mels] (n = st.need())
    through the subsampling and every layer with the caches; returns [q, d_out]."""
    M = st.M
    x = ss_stream_step(M["ss"], st, mel, is_last)
    Q, d = x.shape
    pe = pos_emb(st.valid + Q, d)
    for li, L in enumerate(M["layers"]):
        x = (x + f32(0.5) * half_ffn(L, x, 0)).astype(f32)
        xn = layer_norm(x, L["ln_att_w"], L["ln_att_b"])
        kn, vn = _lin(L, "k_w", xn), _lin(L, "v_w", xn)
        x = (x + _stream_attention(L, xn, kn, vn, pe, M["n_heads"], st.kc[li], st.vc[li])).astype(f32)
        st.kc[li] = np.concatenate([st.kc[li], kn])[-st.left:] if st.left > 0 else np.zeros((0, d), f32)   # update_kv_cache :763-776
        st.vc[li] = np.concatenate([st.vc[li], vn])[-st.left:] if st.left > 0 else np.zeros((0, d), f32)
        y, st.cc[li] = _stream_conv_module(L, layer_norm(x, L["ln_conv_w"], L["ln_conv_b"]), st.cc[li])
        x = (x + y).astype(f32)
        x = (x + f32(0.5) * half_ffn(L, x, 1)).astype(f32)
        x = layer_norm(x, L["ln_out_w"], L["ln_out_b"])
    st.valid = min(st.valid + Q, st.left)
    return encoder_post(M, x, prompt_id)


def stream_encode(M, mel, left, right, prompt_id=0):
    """Feeds valid mel frames through the streaming encoder in the chunk sizes it asks for
    (the loop of mynah_asr_stream_feed, src/mynah_asr.c:868-890); returns the concatenated [T, d_out]."""
    st = EncStream(M, left, right, mel.shape[1])
    outs, pos, T = [], 0, mel.shape[0]
    while pos < T:
        n = st.need()
        outs.append(enc_stream_step(st, mel[pos:pos + n], pos + n >= T, prompt_id))
        pos += n
    return np.concatenate(outs)
