"""Cache-aware streaming encoder on the GPU (lock-step stream groups) against the compiled reference's
streaming outputs (tests/golden/ref_rnnt_kq.npz: mynah_asr_enc_stream_step fed chunk by chunk), the numpy
oracle, and the GPU's own offline limited-context path."""
import os

import numpy as np
import pytest

import cases
from oracle import mynah_oracle as O, model_io

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
NAME = "rnnt_kq"          # Nemotron-style: causal convs, LayerNorm conv norm


def rel(a, b):
    return float(np.linalg.norm(a.astype(np.float64) - b.astype(np.float64)) / max(np.linalg.norm(b), 1e-30))


@pytest.fixture(scope="module")
def setup(gpu_pkg, synth):
    cfg, tensors = cases.build(synth, NAME)
    dm = cases.device_model(gpu_pkg, synth, cfg, tensors)
    mels = []
    for seed in (7, 21, 22):                       # stream 0 is the golden utterance
        feats, valid = dm.log_mel(synth.synth_audio(2.0, seed=seed))
        mels.append(feats[:valid])
    yield cfg, tensors, dm, mels, np.load(os.path.join(GOLD, f"ref_{NAME}.npz"))
    dm.close()


def run_group(dm, mels, left, right):
    g = dm.stream_open(len(mels), left, right)
    outs, pos, T = [], 0, mels[0].shape[0]
    while pos < T:
        n = g.need()
        chunk = np.stack([m[pos:pos + n] for m in mels])
        outs.append(g.step(chunk, pos + n >= T))
        pos += n
    g.close()
    return np.concatenate(outs, axis=1)            # [streams, T, d_out]


@pytest.mark.parametrize("left,right", cases.STREAM_CONTEXTS)
def test_streams_match_reference_and_oracle(setup, left, right):
    cfg, tensors, dm, mels, g = setup
    out = run_group(dm, mels, left, right)
    ref = g[f"stream_{left}_{right}"]
    assert out.shape[1:] == ref.shape
    # tolerance of the path (north star): encoder output within relative L2 1e-3
    assert rel(out[0], ref) < 1e-3
    M = model_io.oracle_model(cfg, tensors)
    for s in (1, 2):
        assert rel(out[s], O.stream_encode(M, mels[s], left, right)) < 1e-3


def test_stream_rows_do_not_depend_on_the_group(setup):
    """A stream's output bits are the same alone, in a group of three, and at another position in it."""
    cfg, tensors, dm, mels, g = setup
    left, right = 8, 1
    three = run_group(dm, mels, left, right)
    assert np.array_equal(run_group(dm, mels[:1], left, right)[0], three[0])
    assert np.array_equal(run_group(dm, [mels[2], mels[0]], left, right)[1], three[0])


def test_group_size_classes(setup):
    """Groups of at most 128 rows per step (streams x frames per chunk) run the linears of their layers on the few-row
    kernel, larger groups on the many-row kernel: inside a class a stream's bits depend neither on the group's size nor
    on its place in the group; across the two classes the outputs agree to f32 rounding (both kernels sum the same
    three fp16 products per term, in different orders)."""
    cfg, tensors, dm, mels, g = setup
    left, right = 8, 1                                                    # two frames per chunk: 64 streams = 128 rows
    small = run_group(dm, mels, left, right)
    edge = run_group(dm, [mels[1]] * 63 + [mels[0]], left, right)         # 64 streams: still the few-row class
    assert np.array_equal(edge[63], small[0]) and np.array_equal(edge[5], small[1])
    big = run_group(dm, [mels[1]] * 64 + [mels[0]], left, right)          # 65 streams: the many-row class
    bigger = run_group(dm, [mels[0]] + [mels[2]] * 70, left, right)
    assert np.array_equal(big[64], bigger[0])
    assert rel(big[64], small[0]) < 1e-5 and rel(big[0], small[1]) < 1e-5


def test_streaming_equals_offline_tokens(setup):
    """Streaming ~ the offline limited-context encoder on the same frames, and the greedy tokens are identical
    (the reference's tests/test_streaming.c checks text equality)."""
    cfg, tensors, dm, mels, g = setup
    for left, right in ((6, 0), (8, 1)):
        out = run_group(dm, mels, left, right)
        for s in range(3):
            off = dm.encoder_forward(mels[s], left=left, right=right)
            assert off.shape == out[s].shape and rel(out[s], off) < 1e-3
            ts, fs = dm.greedy_decode(out[s])
            to, fo = dm.greedy_decode(off)
            assert list(ts) == list(to) and list(fs) == list(fo)


def test_chunkwise_decode_with_carried_state(setup):
    """Greedy RNNT chunk by chunk with the transducer state kept on the device == greedy decode of the whole
    streamed encoder output at once (tokens and absolute frames), for streams in different decode groups."""
    cfg, tensors, dm, mels, g = setup
    left, right = 8, 1
    many = [mels[i % 3] for i in range(19)]                 # 19 streams: two lock-step decode groups
    enc = run_group(dm, many, left, right)
    grp = dm.stream_open(len(many), left, right)
    toks = [[] for _ in many]
    frs = [[] for _ in many]
    pos, T = 0, many[0].shape[0]
    while pos < T:
        n = grp.need()
        res = grp.step_decode(np.stack([m[pos:pos + n] for m in many]), pos + n >= T)
        for s, (t, f) in enumerate(res):
            toks[s] += list(t); frs[s] += list(f)
        pos += n
    grp.close()
    for s in range(len(many)):
        t, f = dm.greedy_decode(enc[s])
        assert toks[s] == list(t) and frs[s] == list(f), s
    assert any(len(t) > 3 for t in toks)


def test_incremental_mel_equals_offline_and_feeds_the_stream(setup, synth):
    """Audio fed in 600-sample pieces (as the reference's tests/test_streaming.c does): the incremental
    log-mel frames are bit-identical to the offline front end, and chunks cut from them as they arrive drive
    the streaming encoder to the same output as chunks cut from the offline frames."""
    cfg, tensors, dm, mels, g = setup
    left, right = 6, 0
    audios = np.stack([synth.synth_audio(2.0, seed=s) for s in (7, 21)])
    grp = dm.stream_open(2, left, right)
    got, pend, outs = [], np.zeros((2, 0, cfg.n_mels), np.float32), []
    total, valid = audios.shape[1], audios.shape[1] // 160
    for pos in range(0, total, 600):
        piece = audios[:, pos:pos + 600]
        fr = grp.mel_feed(piece, finish=pos + 600 >= total)
        got.append(fr)
        pend = np.concatenate([pend, fr], axis=1)
        done = sum(f.shape[1] for f in got)
        while pend.shape[1] >= grp.need() or (done >= valid and pend.shape[1] > 0):
            n = min(grp.need(), pend.shape[1])
            last = done >= valid and pend.shape[1] <= n
            outs.append(grp.step(pend[:, :n], last))
            pend = pend[:, n:]
    grp.close()
    feats = np.concatenate(got, axis=1)
    assert feats.shape[1] == valid
    for s in range(2):
        assert np.array_equal(feats[s], mels[s][:valid])          # mels: offline log-mel of seeds 7, 21
    ref = run_group(dm, mels[:2], left, right)
    assert np.array_equal(np.concatenate(outs, axis=1), ref)


def test_stream_edges(setup, gpu_pkg):
    cfg, tensors, dm, mels, g = setup
    grp = dm.stream_open(2, 6, 0)
    assert grp.need() == 1                         # first chunk: 1 + 8 * right mel frames
    out = grp.step(np.stack([m[:1] for m in mels[:2]]))
    assert out.shape == (2, 1, cfg.d_out) and grp.need() == 8
    with pytest.raises(gpu_pkg.BackendError):      # wrong chunk size
        grp.step(np.stack([m[1:4] for m in mels[:2]]))
    grp.close()
    with pytest.raises(gpu_pkg.BackendError):      # chunk longer than the left context
        dm.stream_open(1, 2, 3)
