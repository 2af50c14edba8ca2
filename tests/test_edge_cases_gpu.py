"""Edge cases of the scoring and decoding entry points: empty and ragged minibatches, one-word sentences, columns
that are padding only, the longest sentences the reference's file preparation lets through, hypothesis lists that
come back short.  Every result is compared with the CPU oracle on the same inputs."""
import numpy as np
import pytest

from zoph_rnn_b200 import synth
from tests import helpers

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def api():
    import torch
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    from zoph_rnn_b200 import api as a
    return a


def build(api, cfg, w, dtype):
    m = api.neuralMT_model(cfg, dtype=dtype)
    m.load_weights(w)
    return m


@pytest.mark.parametrize("dtype", [3, 5])
def test_ragged_minibatch_with_padding_only_columns(api, oracle, dtype):
    """Sentences of length 1 next to the longest ones, and two columns that hold nothing but -1 (the filler rows the
    reference appends to complete a minibatch): their log-probs are exactly 0 and the other columns are unaffected."""
    cfg = synth.make_cfg(2, 128, 90, 120, attention=1, feed_input=1, D=2)
    w = synth.make_weights(cfg, seed=51, scale=0.2)
    rng = np.random.default_rng(3)
    B, S, T = 9, 13, 15
    src = np.full((S, B), -1, np.int32)
    tin = np.full((T, B), -1, np.int32)
    tout = np.full((T, B), -1, np.int32)
    lens_s = [13, 1, 7, 1, 13, 2, 5, 0, 0]
    lens_t = [14, 1, 1, 14, 6, 2, 9, 0, 0]   # number of target words (the rows hold len + 1 ids)
    for b in range(B):
        if lens_s[b] == 0:
            continue
        src[S - lens_s[b]:, b] = rng.integers(0, 90, lens_s[b])
        y = rng.integers(3, 120, lens_t[b])
        tin[:lens_t[b] + 1, b] = np.concatenate([[0], y])
        tout[:lens_t[b] + 1, b] = np.concatenate([y, [1]])
    # padding-only columns still need one source id for the reference's layout; the oracle and the library treat a
    # column without any source word as length 0, so give them a single <UNK> and an all -1 target
    src[S - 1, 7:] = 0
    want = oracle.OracleModel(cfg, w).score_batch(src, tin, tout)
    got, total = build(api, cfg, w, dtype).get_error(src, tin, tout)
    helpers.assert_logp_close(got, want, rtol=2e-5, atol=3e-6)
    assert np.all(got[:, 7:] == 0.0)
    assert abs(total - want.sum()) < 1e-4 * abs(want.sum())


@pytest.mark.parametrize("dtype", [3, 5])
def test_single_column_single_step(api, oracle, dtype):
    cfg = synth.make_cfg(1, 128, 0, 64, lm=True)
    w = synth.make_weights(cfg, seed=52, scale=0.3)
    tin = np.array([[0]], np.int32)
    tout = np.array([[1]], np.int32)
    want = oracle.OracleModel(cfg, w).score_batch(None, tin, tout)
    got, _ = build(api, cfg, w, dtype).get_error(None, tin, tout)
    helpers.assert_logp_close(got, want, rtol=2e-5, atol=3e-6)


def test_empty_minibatch_is_a_no_op(api):
    cfg = synth.make_cfg(1, 128, 0, 64, lm=True)
    m = build(api, cfg, synth.make_weights(cfg, seed=53), 0)
    lp, total = m.get_error(None, np.zeros((0, 4), np.int32), np.zeros((0, 4), np.int32))
    assert lp.size == 0 and total == 0.0
    ids, ln, sc = build(api, synth.make_cfg(1, 128, 50, 64), synth.make_weights(synth.make_cfg(1, 128, 50, 64), seed=54),
                        0).decode([], beam=4)
    assert ids.shape[0] == 0 and ln.shape[0] == 0


@pytest.mark.parametrize("dtype", [3, 5])
def test_longest_sentences_the_file_preparation_keeps(api, oracle, dtype):
    """-L 100: the reference keeps sentences with len + 1 < L - 2, i.e. up to 96 words (97 target positions)."""
    cfg = synth.make_cfg(1, 128, 300, 300, attention=1, feed_input=1, D=10)
    w = synth.make_weights(cfg, seed=55, scale=0.15)
    src, tin, tout = synth.make_s2s_batch(300, 300, 3, 96, 96, 96, 96, seed=8)
    assert src.shape[0] == 96 and tin.shape[0] >= 96
    want = oracle.OracleModel(cfg, w).score_batch(src, tin, tout)
    got, _ = build(api, cfg, w, dtype).get_error(src, tin, tout)
    helpers.assert_logp_close(got, want, rtol=3e-5, atol=3e-6)


@pytest.mark.parametrize("dtype", [3, 5])
def test_decode_limits_and_short_hypothesis_lists(api, oracle, dtype):
    """One-word sources (the step limit (int)(max_ratio * S) is 1), a k-best request larger than the number of
    finished hypotheses, and a min ratio that filters everything: lengths of 0 mark the missing entries."""
    cfg = synth.make_cfg(1, 128, 80, 100, attention=1, feed_input=1, D=2)
    w = synth.make_weights(cfg, seed=56, scale=0.3)
    srcs = [np.array([5], np.int32), np.array([7, 9], np.int32), np.array([3], np.int32)]
    om = oracle.OracleModel(cfg, w)
    m = build(api, cfg, w, dtype)
    short = 0
    for kw in (dict(beam=3, k_best=8, min_ratio=0.5, max_ratio=1.5, penalty=0.0, longest_sent=20),
               dict(beam=3, k_best=2, min_ratio=50.0, max_ratio=60.0, penalty=0.0, longest_sent=20),
               dict(beam=9, k_best=3, min_ratio=0.0, max_ratio=40.0, penalty=0.5, longest_sent=6)):
        ids, ln, sc = om.beam_decode(srcs, **kw)
        gi, gl, gs = m.decode(srcs, **kw)
        assert np.array_equal(gl, ln), (kw, gl, ln)
        assert np.array_equal(gi, ids)
        np.testing.assert_allclose(gs[ln > 0], sc[ln > 0], rtol=1e-5, atol=1e-4)
        short += int((ln == 0).sum())
    assert short > 0  # the first two settings leave k-best slots empty


@pytest.mark.parametrize("att,lm,L,H,Vs,Vt,B,S,T", [
    (1, 0, 1, 132, 333, 1003, 1, (7, 7), (9, 9)),        # one column, hidden size off the 64-element padding
    (2, 0, 2, 260, 97, 257, 129, (2, 6), (2, 5)),        # one column more than a 128-row tile
    (0, 1, 3, 1020, 0, 5001, 200, (0, 0), (3, 8)),       # language model, two row tiles, odd vocabulary
    (1, 0, 1, 512, 64, 129, 7, (1, 30), (1, 3)),         # vocabulary just above one softmax tile
    (2, 0, 1, 128, 50, 31, 3, (4, 4), (6, 6)),           # vocabulary smaller than any tile
    (2, 0, 8, 64, 40, 90, 5, (1, 9), (2, 4)),            # eight layers: the widest multi-cell encoder launch
    (1, 0, 3, 1000, 60, 120, 20, (2, 7), (2, 3)),        # three layers of 32 row tiles: encoder diagonals, K unsplit
    (2, 0, 5, 1000, 60, 120, 9, (3, 3), (2, 2)),         # five such layers do not fit the SMs: layer-by-layer encoder
])
def test_shape_sweep_against_the_oracle(api, oracle, att, lm, L, H, Vs, Vt, B, S, T):
    """Shapes around the kernels' tile boundaries, fp32-accurate tensor-core engine and the bf16 engine."""
    cfg = synth.make_cfg(L, H, Vs, Vt, lm=bool(lm), attention=att, feed_input=1 if att else 0, D=3)
    w = synth.make_weights(cfg, seed=60 + H, scale=0.1)
    if lm:
        tin, tout = synth.make_lm_batch(Vt, B, T[1], seed=5)
        src = None
    else:
        src, tin, tout = synth.make_s2s_batch(Vs, Vt, B, S[0], S[1], T[0], T[1], seed=5)
    want = oracle.OracleModel(cfg, w).score_batch(src, tin, tout)
    got, _ = build(api, cfg, w, 5).get_error(src, tin, tout)
    helpers.assert_logp_close(got, want, rtol=2e-5, atol=3e-6)
    if H % 8 == 0:
        got16, _ = build(api, cfg, w, 1).get_error(src, tin, tout)
        msk = tout != -1
        assert np.abs(got16[msk] - want[msk]).max() < 0.08
        assert abs(got16[msk].sum() - want[msk].sum()) < 5e-3 * abs(want[msk].sum())


def test_two_devices_in_one_process(api):
    """zrnn_set_device lets one process put models on several devices in turn: per-device state inside the library
    (kernel attributes, error word, scratch addresses) must not leak from one device to the other."""
    import ctypes
    import torch
    n = ctypes.c_int()
    api.check(api.lib().zrnn_device_count(ctypes.byref(n)))
    assert n.value == torch.cuda.device_count()
    if n.value < 2:
        pytest.skip("needs two devices")
    cfg = synth.make_cfg(2, 256, 300, 400, attention=2, feed_input=1)
    w = synth.make_weights(cfg, seed=70, scale=0.1)
    src, tin, tout = synth.make_s2s_batch(300, 400, 8, 4, 12, 4, 12, seed=6)
    results = []
    try:
        for dev in (0, 1):
            api.check(api.lib().zrnn_set_device(dev))
            torch.cuda.set_device(dev)
            m = build(api, cfg, w, 0)
            results.append(m.get_error(src, tin, tout)[0])
            del m
    finally:
        api.check(api.lib().zrnn_set_device(0))
        torch.cuda.set_device(0)
    assert np.array_equal(results[0], results[1])
