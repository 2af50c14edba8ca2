"""Error paths on the device: a bounded wait that runs out, beam widths at and beyond the limit."""
import ctypes

import numpy as np
import pytest

from zoph_rnn_b200 import synth

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def api():
    from zoph_rnn_b200 import api as a
    return a


def small_model(api, dtype=3, V=1500):
    cfg = synth.make_cfg(1, 64, 200, V, attention=2, feed_input=1)
    w = synth.make_weights(cfg, seed=3, scale=0.2)
    m = api.neuralMT_model(cfg, dtype=dtype)
    m.load_weights(w)
    return cfg, w, m


def test_bounded_wait_runs_out_and_the_context_survives(api):
    """A device wait on a barrier that nothing completes gives up after its limit (here about a millisecond), the
    kernel returns, the error word holds the waiting role, the next synchronising call reports ZRNN_E_TIMEOUT once,
    and the call after that succeeds with correct results."""
    import torch
    cfg, w, m = small_model(api)
    src, tin, tout = synth.make_s2s_batch(200, 1500, 3, 2, 5, 3, 4, seed=1)
    want, _ = m.get_error(src, tin, tout)
    assert api.lib().zrnn_tc_error() == 0
    api.check(api.lib().zrnn_debug_bounded_wait(2_000_000, None))
    torch.cuda.synchronize()  # the kernel came back by itself
    assert api.lib().zrnn_tc_error() == 77
    assert api.lib().zrnn_tc_error() == 0  # reading clears it
    api.check(api.lib().zrnn_debug_bounded_wait(2_000_000, None))
    with pytest.raises(api.ZrnnError) as e:
        m.get_error(src, tin, tout)
    assert e.value.status == 4 and "bounded device wait" in str(e.value)
    got, _ = m.get_error(src, tin, tout)
    np.testing.assert_array_equal(got, want)
    with pytest.raises(api.ZrnnError):
        api.check(api.lib().zrnn_debug_bounded_wait(0, None))


@pytest.mark.parametrize("beam", [16, 24, 32])
def test_wide_beams_match_the_oracle(api, oracle, beam):
    cfg, w, m = small_model(api)
    srcs = synth.make_decode_sources(200, 6, 3, 8, seed=4)
    kw = dict(beam=beam, k_best=3, min_ratio=0.5, max_ratio=2.0, penalty=0.0, longest_sent=30)
    ids, ln, sc = oracle.OracleModel(cfg, w).beam_decode(srcs, **kw)
    gi, gl, gs = m.decode(srcs, **kw)
    np.testing.assert_array_equal(gl, ln)
    np.testing.assert_array_equal(gi, ids)
    np.testing.assert_allclose(gs, sc, rtol=1e-4, atol=1e-4)


def test_beam_beyond_the_limit_is_rejected(api):
    cfg, w, m = small_model(api)
    srcs = [np.array([5, 6, 7], np.int32)]
    with pytest.raises(api.ZrnnError) as e:
        m.decode(srcs, beam=33, longest_sent=10)
    assert e.value.status == 1 and "beam" in str(e.value)
    # the sqrt(V) cap of the reference applies first: a beam of 100 on a 900-word vocabulary is a beam of 30
    # (and beam 16 .. 32 on the 1500-word vocabulary above are what they say: sqrt(1500) = 38)
    cfg2, w2, m2 = small_model(api, V=900)
    ids, ln, sc = m2.decode(srcs, beam=100, longest_sent=10)
    assert ln[0, 0] > 0


def test_topk_of_33(api, oracle):
    import torch
    rng = np.random.default_rng(0)
    V, H, N, k = 5000, 64, 40, 33
    D = (rng.standard_normal(V * H) / np.sqrt(H)).astype(np.float32)
    b = (rng.standard_normal(V) * 0.1).astype(np.float32)
    h = (rng.standard_normal(H * N) * 2).astype(np.float32)
    p = oracle.softmax_dist(V, H, N, D, b, h).reshape(N, V)
    order = np.argsort(-p, axis=1, kind="stable")[:, :k]
    sm = api.softmax_layer(V, H, dtype=3)
    sm.load_weights(D, b)
    val, idx, eos = sm.topk(torch.as_tensor(h).cuda(), k)
    np.testing.assert_array_equal(idx.cpu().numpy(), order)
    np.testing.assert_allclose(np.exp(val.cpu().numpy().astype(np.float64)), np.take_along_axis(p, order, axis=1), rtol=1e-4)
    with pytest.raises(api.ZrnnError):
        sm.topk(torch.as_tensor(h).cuda(), 34)
