"""The persistent decoder kernel (csrc/tc_decoder.cu): the whole target side of a feed-input model in one launch.
It is opt-in (environment ZRNN_PERSISTENT=1, read at every call); these tests switch it on and compare the scoring
pass with the oracle, with the default per-launch path, and across the ways the kernel can cut the batch into column
groups."""
import os

import numpy as np
import pytest

from tests import helpers
from zoph_rnn_b200 import synth

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def api():
    import torch
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    from zoph_rnn_b200 import api as a
    return a


@pytest.fixture()
def persistent():
    old = {k: os.environ.get(k) for k in ("ZRNN_PERSISTENT", "ZRNN_DEC_GROUPS")}
    os.environ["ZRNN_PERSISTENT"] = "1"
    yield
    for k, v in old.items():
        if v is None:
            os.environ.pop(k, None)
        else:
            os.environ[k] = v


# (attention type, layers, H, B, source lengths, target lengths): one and several row tiles per cluster, fewer k-blocks
# than CTAs (H = 96 in bf16), ragged sources with masks, a batch that is not a multiple of the group size
SHAPES = [(2, 4, 96, 16, (12, 12), (11, 11)), (1, 2, 128, 16, (5, 40), (4, 20)), (2, 2, 256, 37, (3, 9), (3, 9)),
          (1, 1, 200, 128, (4, 6), (5, 5)), (2, 4, 1000, 24, (20, 20), (12, 12))]


@pytest.mark.parametrize("dtype", [4, 5])
@pytest.mark.parametrize("att,L,H,B,S,T", SHAPES)
def test_persistent_decoder_matches_oracle(api, oracle, persistent, att, L, H, B, S, T, dtype):
    cfg = synth.make_cfg(L, H, 500, 700, attention=att, feed_input=1, D=10)
    w = synth.make_weights(cfg, seed=42, scale=0.1)
    src, tin, tout = synth.make_s2s_batch(500, 700, B, S[0], S[1], T[0], T[1], seed=7)
    want = oracle.OracleModel(cfg, w).score_batch(src, tin, tout)
    m = api.neuralMT_model(cfg, dtype=dtype)
    m.load_weights(w)
    for groups in ("1", "2", "4"):
        os.environ["ZRNN_DEC_GROUPS"] = groups
        api.reset_launch_count()
        for _ in range(3):  # eager pass, graph capture, graph replay
            lp, _ = m.get_error(src, tin, tout)
            helpers.assert_logp_close(lp, want)
        assert api.lib().zrnn_tc_error() == 0
    # the kernel really ran: far fewer launches than the L + 2 per target step of the per-launch path
    os.environ["ZRNN_PERSISTENT"] = "0"
    api.reset_launch_count()
    base, _ = m.get_error(src, tin, tout)
    n_plain = api.launch_count()
    os.environ["ZRNN_PERSISTENT"] = "1"
    api.reset_launch_count()
    again, _ = m.get_error(src, tin, tout)
    assert api.launch_count() < n_plain - tin.shape[0] * L
    helpers.assert_logp_close(again, base, rtol=2e-5, atol=2e-6)


@pytest.mark.parametrize("dtype", [1, 2])
def test_persistent_decoder_reduced_precision(api, oracle, persistent, dtype):
    cfg = synth.make_cfg(2, 256, 2000, 3000, attention=2, feed_input=1)
    w = synth.make_weights(cfg, seed=33, scale=0.1)
    src, tin, tout = synth.make_s2s_batch(2000, 3000, 32, 5, 20, 5, 20, seed=11)
    want = oracle.OracleModel(cfg, w).score_batch(src, tin, tout)
    m = api.neuralMT_model(cfg, dtype=dtype)
    m.load_weights(w)
    lp, _ = m.get_error(src, tin, tout)
    n = (tout != -1).sum()
    ppl_got, ppl_want = np.exp(-lp.sum() / n), np.exp(-want.sum() / n)
    assert abs(ppl_got - ppl_want) / ppl_want < 5e-3
    assert np.abs(lp - want).max() < 0.05
