"""Parity at the sizes the benchmark numbers are quoted on (the five workload shapes at full layer and vocabulary
sizes, on a bounded number of sentences so that the CPU oracle finishes in seconds), plus the accuracy gates of the
reduced-precision tensor-core paths: perplexity within 0.5 % and greedy / beam token agreement >= 99.5 %.
"""
import numpy as np
import pytest

from tests import helpers
from zoph_rnn_b200 import synth

pytestmark = pytest.mark.gpu

F32, BF16, TF32, F32_SIMT, F32_3XTF32, F32_F16X2 = range(6)


@pytest.fixture(scope="module")
def api():
    import torch
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    from zoph_rnn_b200 import api as a
    return a


def build_model(api, cfg, w, dtype):
    m = api.neuralMT_model(cfg, dtype=dtype)
    m.load_weights(w)
    return m


def ppl(lp, tout):
    n = (tout != -1).sum()
    return float(np.exp(-np.asarray(lp, dtype=np.float64).sum() / n))


# ---------------------------------------------------------------------------------------------------------------
# configuration 2: seq2seq 4 x 1000, V = 50k / 50k, S = T = 50, global-dot attention + feed-input
# ---------------------------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def config2(oracle):
    cfg = synth.make_cfg(4, 1000, 50000, 50000, attention=2, feed_input=1)
    w = synth.make_weights(cfg, seed=1234, scale=0.1)
    src, tin, tout = synth.make_s2s_batch(50000, 50000, 8, 50, 50, 50, 50, seed=1234, zipf_s=1.1)
    want = oracle.OracleModel(cfg, w).score_batch(src, tin, tout)
    return cfg, w, src, tin, tout, want


@pytest.mark.parametrize("dtype", [F32_3XTF32, F32_F16X2])
def test_config2_full_size_logprobs(api, config2, dtype):
    """fp32-accurate engines on the full 4 x 1000 / V = 50k model over 50 + 50 steps: per-token log-probs within 1e-5."""
    cfg, w, src, tin, tout, want = config2
    m = build_model(api, cfg, w, dtype)
    lp, tot = m.get_error(src, tin, tout)
    helpers.assert_logp_close(lp, want)
    assert abs(tot - want.sum()) < 1e-5 * abs(want.sum())


@pytest.mark.parametrize("dtype", [BF16, TF32])
def test_config2_full_size_reduced_precision_perplexity(api, config2, dtype):
    """bf16 / tf32 tensor-core paths (tanh.approx activations) over the full depth: perplexity within 0.5 %."""
    cfg, w, src, tin, tout, want = config2
    m = build_model(api, cfg, w, dtype)
    lp, _ = m.get_error(src, tin, tout)
    assert abs(ppl(lp, tout) - ppl(want, tout)) / ppl(want, tout) < 5e-3


# ---------------------------------------------------------------------------------------------------------------
# configuration 3: seq2seq 2 x 1000, V = 40k / 40k, ragged sources 10..80, T = 60, local-p D = 10 + feed-input
# ---------------------------------------------------------------------------------------------------------------
def test_config3_full_size_logprobs(api, oracle):
    cfg = synth.make_cfg(2, 1000, 40000, 40000, attention=1, feed_input=1, D=10)
    w = synth.make_weights(cfg, seed=1234, scale=0.1)
    src, tin, tout = synth.make_s2s_batch(40000, 40000, 8, 10, 80, 60, 60, seed=1234, zipf_s=1.1)
    want = oracle.OracleModel(cfg, w).score_batch(src, tin, tout)
    for dtype in (F32_F16X2, F32_3XTF32):
        lp, _ = build_model(api, cfg, w, dtype).get_error(src, tin, tout)
        helpers.assert_logp_close(lp, want)
    lp, _ = build_model(api, cfg, w, BF16).get_error(src, tin, tout)
    assert abs(ppl(lp, tout) - ppl(want, tout)) / ppl(want, tout) < 5e-3


# ---------------------------------------------------------------------------------------------------------------
# configuration 4: beam 12 decode, 2 x 1000, V = 50k, global attention
# ---------------------------------------------------------------------------------------------------------------
def test_config4_full_size_beam_decode(api, oracle):
    """Three sentences through the full-size decoder: every hypothesis equals the oracle's token for token (the
    weights are random, so hypotheses run to the length limit: ~100 beam steps each)."""
    cfg = synth.make_cfg(2, 1000, 50000, 50000, attention=2, feed_input=1)
    w = synth.make_weights(cfg, seed=1234, scale=0.1)
    srcs = synth.make_decode_sources(50000, 3, 10, 50, seed=5, zipf_s=1.1)
    kw = dict(beam=12, k_best=1, min_ratio=0.5, max_ratio=2.0, penalty=0.0, longest_sent=100)
    ids, ln, sc = oracle.OracleModel(cfg, w).beam_decode(srcs, **kw)
    for dtype in (F32_F16X2, F32_3XTF32):
        gi, gl, gs = build_model(api, cfg, w, dtype).decode(srcs, **kw)
        assert np.array_equal(gl, ln)
        assert np.array_equal(gi, ids)
        np.testing.assert_allclose(gs, sc, rtol=1e-5, atol=1e-4)


# ---------------------------------------------------------------------------------------------------------------
# configuration 5: LM 2 x 2048, V = 200k, N(0, 0.02) weights, specified in bf16
# ---------------------------------------------------------------------------------------------------------------
def test_config5_full_size_bf16(api, oracle):
    """8 sentences x 16 steps of the 2 x 2048 / V = 200k model.  The weights are rounded to bf16 first (the
    configuration stores them in bf16), so the oracle computes in fp32 on exactly the values the tensor cores see and the
    remaining difference is the bf16 rounding of the activations and the approximate tanh: perplexity within 0.5 %."""
    cfg = synth.make_cfg(2, 2048, 0, 200000, lm=1)
    w = synth.make_weights(cfg, seed=1234, dist="normal", scale=0.02, round_bf16=True)
    tin, tout = synth.make_lm_batch(200000, 8, 16, seed=1234, zipf_s=1.05)
    want = oracle.OracleModel(cfg, w).score_batch(None, tin, tout)
    lp, _ = build_model(api, cfg, w, BF16).get_error(None, tin, tout)
    assert abs(ppl(lp, tout) - ppl(want, tout)) / ppl(want, tout) < 5e-3
    assert np.abs(lp - want).max() < 0.05
    # and the fp32-accurate engine on the same model at 1e-5
    lp, _ = build_model(api, cfg, w, F32_F16X2).get_error(None, tin, tout)
    helpers.assert_logp_close(lp, want)


# ---------------------------------------------------------------------------------------------------------------
# reduced-precision paths: token agreement of greedy and beam decoding
# ---------------------------------------------------------------------------------------------------------------
# A decision counts as a near-tie when the oracle itself was this close to deciding otherwise.  Greedy: the chosen
# word leads the runner-up by less than twice the per-token log-prob deviation the perplexity tests allow (0.05), so
# a deviation inside that bound cannot flip a decision that is not a near-tie.  Beam: the best and the second-best
# finished hypotheses score within 0.5 nats of each other (scores are sums over up to ~20 tokens).
NEAR_TIE_NATS = 0.1
NEAR_TIE_BEAM_NATS = 0.5


def greedy_gaps(oracle, om, cfg, w, src_rev, hyp):
    """Per step of the oracle's greedy hypothesis `hyp` (<START> y1 .. yn <EOF>) the gap (nats) between the chosen
    word and the runner-up: the oracle is run teacher-forced along its own hypothesis and the full output distribution
    of every step is formed from the vectors it hands to the softmax."""
    y = np.asarray(hyp, dtype=np.int32)
    tin, tout = y[:-1].reshape(-1, 1), y[1:].reshape(-1, 1)
    src = np.asarray(src_rev, dtype=np.int32).reshape(-1, 1)
    _, top = om.score_batch(src, tin, tout, want_top=True)
    T, V, H = tin.shape[0], cfg["V_tgt"], cfg["H"]
    _, allp = oracle.softmax_logp(V, H, T, w[-2], w[-1], top.reshape(T, H), tout.reshape(-1), want_all=True)
    allp = allp.reshape(T, V).copy()
    allp[:, 0] = -np.inf  # <START> is never expanded (src/decoder.h:1255)
    part = np.partition(allp, V - 2, axis=1)
    return part[:, V - 1] - part[:, V - 2]


@pytest.mark.parametrize("dtype,name", [(BF16, "bf16"), (TF32, "tf32")])
def test_reduced_precision_token_agreement(api, oracle, dtype, name):
    """Greedy (beam 1) and beam-12 decodes of the bf16 / tf32 paths against the oracle: >= 99.5 % of the tokens agree
    once near-ties are set aside.  Greedy: every sentence counts up to its first near-tie step (after a flipped
    decision the two decoders follow different prefixes).  Beam 12: sentences whose two best hypotheses are a near-tie
    are left out."""
    cfg = synth.make_cfg(2, 256, 2000, 3000, attention=2, feed_input=1)
    w = synth.make_weights(cfg, seed=33, scale=0.5)  # large weights: peaked output distributions
    srcs = synth.make_decode_sources(2000, 64, 3, 10, seed=12)
    om = oracle.OracleModel(cfg, w)
    m = build_model(api, cfg, w, dtype)
    # ---- greedy
    kw = dict(beam=1, k_best=1, min_ratio=0.0, max_ratio=2.0, penalty=0.0, longest_sent=40)
    ids, ln, _ = om.beam_decode(srcs, **kw)
    gi, gl, _ = m.decode(srcs, **kw)
    same = total = 0
    for i in range(len(srcs)):
        n = int(ln[i, 0])
        if n < 2:
            continue
        gaps = greedy_gaps(oracle, om, cfg, w, srcs[i], ids[i, 0, :n])
        ties = np.nonzero(gaps < NEAR_TIE_NATS)[0]
        cut = int(ties[0]) if len(ties) else n - 1  # decisions 0 .. cut-1 are clear; decision t yields token t+1
        same += int((ids[i, 0, 1:1 + cut] == gi[i, 0, 1:1 + cut]).sum())
        total += cut
    assert total >= 150, f"{name} greedy: only {total} clear decisions"
    assert same / total >= 0.995, f"{name} greedy: token agreement {same / total:.4f} over {total} tokens"
    # ---- beam 12
    kw = dict(beam=12, k_best=2, min_ratio=0.0, max_ratio=2.0, penalty=0.0, longest_sent=40)
    ids, ln, sc = om.beam_decode(srcs, **kw)
    gi, gl, _ = m.decode(srcs, **kw)
    keep = [i for i in range(len(srcs))
            if ln[i, 0] > 0 and not (ln[i, 1] > 0 and abs(float(sc[i, 0]) - float(sc[i, 1])) < NEAR_TIE_BEAM_NATS)]
    assert len(keep) >= len(srcs) // 4, f"{name} beam 12: only {len(keep)} sentences without a near-tie"
    same = total = 0
    for i in keep:
        n = max(int(ln[i, 0]), int(gl[i, 0]))
        same += int((ids[i, 0, :n] == gi[i, 0, :n]).sum())
        total += n
    assert same / total >= 0.995, f"{name} beam 12: token agreement {same / total:.4f} over {len(keep)} sentences"


@pytest.mark.parametrize("dtype,name", [(BF16, "bf16"), (TF32, "tf32")])
def test_reduced_precision_perplexity_deep_and_long(api, oracle, dtype, name):
    """The approximate activations compound over layers and steps: 4 layers x 50 + 50 steps, H = 512."""
    cfg = synth.make_cfg(4, 512, 3000, 3000, attention=1, feed_input=1, D=10)
    w = synth.make_weights(cfg, seed=35, scale=0.1)
    src, tin, tout = synth.make_s2s_batch(3000, 3000, 16, 30, 50, 50, 50, seed=13)
    want = oracle.OracleModel(cfg, w).score_batch(src, tin, tout)
    lp, _ = build_model(api, cfg, w, dtype).get_error(src, tin, tout)
    assert abs(ppl(lp, tout) - ppl(want, tout)) / ppl(want, tout) < 5e-3, name
    assert np.abs(lp - want).max() < 0.05


# ---------------------------------------------------------------------------------------------------------------
# weights reloaded between scoring passes (how get_perplexity is used during training)
# ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [F32_SIMT, F32_F16X2])
def test_reload_weights_after_graph_capture(api, oracle, dtype):
    """Three passes with the same shapes (the second captures a CUDA graph, the third replays it), then new weights,
    then the same call again: the pass must use the new weights, not a graph over the freed buffers."""
    cfg = synth.make_cfg(2, 128, 300, 400, attention=2, feed_input=1)
    src, tin, tout = synth.make_s2s_batch(300, 400, 6, 4, 9, 4, 9, seed=5)
    w1 = synth.make_weights(cfg, seed=1, scale=0.2)
    w2 = synth.make_weights(cfg, seed=2, scale=0.2)
    m = build_model(api, cfg, w1, dtype)
    want1 = oracle.OracleModel(cfg, w1).score_batch(src, tin, tout)
    for _ in range(3):
        lp, _ = m.get_error(src, tin, tout)
        helpers.assert_logp_close(lp, want1)
    m.load_weights(w2)
    want2 = oracle.OracleModel(cfg, w2).score_batch(src, tin, tout)
    for _ in range(3):
        lp, _ = m.get_error(src, tin, tout)
        helpers.assert_logp_close(lp, want2)


def test_partial_weight_update(api, oracle):
    """After the first finalize a layer is re-loaded as a whole: setting one tensor of it and finalizing is a call
    order error that names a missing tensor; setting all tensors of one layer updates that layer only."""
    import ctypes
    from zoph_rnn_b200 import _lib
    cfg = synth.make_cfg(2, 64, 0, 200, lm=1)
    w1 = synth.make_weights(cfg, seed=1, scale=0.2)
    w2 = synth.make_weights(cfg, seed=2, scale=0.2)
    tin, tout = synth.make_lm_batch(200, 5, 7, seed=3)
    m = build_model(api, cfg, w1, F32_SIMT)
    spec = m.tensor_spec()

    def set_tensor(i, t):
        t = np.ascontiguousarray(t, dtype=np.float32).reshape(-1)
        api.check(api.lib().zrnn_model_set_tensor(m._h, i, t.ctypes.data_as(_lib.c_float_p)))
    set_tensor(0, w2[0])
    with pytest.raises(api.ZrnnError) as e:
        api.check(api.lib().zrnn_model_finalize(m._h))
    assert e.value.status == 6 and "must be set again" in str(e.value)
    with pytest.raises(api.ZrnnError) as e:  # the model stays unusable until the update is completed
        m.get_error(None, tin, tout)
    assert e.value.status == 6
    # complete the update of layer 0 (every tensor whose name starts with tgt0.)
    mixed = list(w1)
    for i, (name, _, _) in enumerate(spec):
        if name.startswith("tgt0."):
            set_tensor(i, w2[i])
            mixed[i] = w2[i]
    api.check(api.lib().zrnn_model_finalize(m._h))
    lp, _ = m.get_error(None, tin, tout)
    helpers.assert_logp_close(lp, oracle.OracleModel(cfg, mixed).score_batch(None, tin, tout))


def test_token_ids_outside_the_vocabulary_are_rejected(api):
    """Host id arrays are validated before anything is launched (an id of another vocabulary would index past the
    embedding table)."""
    cfg = synth.make_cfg(1, 32, 50, 60, attention=0)
    m = build_model(api, cfg, synth.make_weights(cfg, seed=1), F32_SIMT)
    src, tin, tout = synth.make_s2s_batch(50, 60, 3, 3, 5, 3, 5, seed=1)
    for which in range(3):
        arrs = [src.copy(), tin.copy(), tout.copy()]
        arrs[which][-1, 1] = 60 if which else 50
        with pytest.raises(api.ZrnnError) as e:
            m.get_error(*arrs)
        assert e.value.status == 1 and "outside the vocabulary" in str(e.value)
    with pytest.raises(api.ZrnnError) as e:
        m.decode([np.array([3, 50], np.int32)], beam=2, longest_sent=10)
    assert e.value.status == 1 and "outside the vocabulary" in str(e.value)
    with pytest.raises(api.ZrnnError) as e:
        m.decode([np.array([3, -2], np.int32)], beam=2, longest_sent=10)
    assert e.value.status == 1
    lp, _ = m.get_error(src, tin, tout)  # the model is still usable
    assert np.isfinite(lp).all()
