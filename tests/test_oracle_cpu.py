"""CPU tests: the oracle against the committed goldens and the NumPy witness, the host-side logic,
and the C-ABI library's exported symbols.  No GPU needed."""
import ctypes
import os
import re

import numpy as np
import pytest

from tests import helpers
from zoph_rnn_b200 import synth

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("name", helpers.golden_cases())
def test_oracle_matches_golden_scores(oracle, name):
    cfg, w, g = helpers.load_golden(name)
    m = oracle.OracleModel(cfg, w)
    src = g["src"] if "src" in g else None
    lp = m.score_batch(src, g["tgt_in"], g["tgt_out"])
    helpers.assert_logp_close(lp, g["logp"], rtol=1e-6, atol=1e-6)
    # padded positions score exactly 0
    assert np.all(lp[g["tgt_out"] == -1] == 0.0)


@pytest.mark.parametrize("name", [n for n in helpers.golden_cases() if n.startswith("s2s")])
def test_oracle_matches_golden_decodes(oracle, name):
    from tests.golden.make_golden import DECODE as d
    cfg, w, g = helpers.load_golden(name)
    m = oracle.OracleModel(cfg, w)
    srcs = helpers.split_sources(g["dec_src"], g["dec_len"])
    ids, ln, sc = m.beam_decode(srcs, d["beam"], d["k_best"], d["min_ratio"], d["max_ratio"], d["penalty"], d["longest_sent"])
    assert np.array_equal(ids, g["dec_ids"])
    assert np.array_equal(ln, g["dec_hyp_len"])
    np.testing.assert_allclose(sc, g["dec_score"], rtol=1e-6, atol=1e-6)


def test_oracle_vs_numpy_witness_fresh_case(oracle):
    from oracle import ref_numpy as rn
    cfg = synth.make_cfg(2, 19, 31, 37, attention=1, feed_input=1, D=2)
    w = synth.make_weights(cfg, seed=77, scale=0.4)
    src, tin, tout = synth.make_s2s_batch(31, 37, 5, 2, 11, 2, 7, seed=5)
    a = oracle.OracleModel(cfg, w).score_batch(src, tin, tout)
    b = rn.score_batch(cfg, w, src, tin, tout)
    helpers.assert_logp_close(a, b, rtol=1e-6, atol=1e-6)


def test_oracle_layer_functions(oracle):
    rng = np.random.default_rng(0)
    H, V, B = 12, 9, 5
    W = rng.standard_normal(H * V).astype(np.float32)
    ids = np.array([3, -1, 8, 0, 3], dtype=np.int32)
    x = oracle.gather(W, H, ids).reshape(B, H)
    Wm = W.reshape(V, H)
    assert np.array_equal(x[0], Wm[3]) and np.array_equal(x[1], Wm[0]) and np.array_equal(x[2], Wm[8])
    # log-softmax sums to one and the decode distribution agrees with it
    D = rng.standard_normal(V * H).astype(np.float32) * 0.3
    b = rng.standard_normal(V).astype(np.float32) * 0.1
    h = rng.standard_normal(H * B).astype(np.float32)
    tgt = np.array([0, 1, 2, 3, 4], dtype=np.int32)
    lp, allp = oracle.softmax_logp(V, H, B, D, b, h, tgt, want_all=True)
    allp = allp.reshape(B, V)
    np.testing.assert_allclose(np.exp(allp).sum(axis=1), 1.0, rtol=1e-12)
    assert np.allclose(lp, allp[np.arange(B), tgt])
    p = oracle.softmax_dist(V, H, B, D, b, h).reshape(B, V)
    np.testing.assert_allclose(np.log(p), allp, rtol=0, atol=2e-6)


def test_masked_columns_are_zero_and_independent(oracle):
    """Padding must not leak: scoring a sentence alone or inside a padded batch gives the same numbers."""
    cfg = synth.make_cfg(2, 16, 29, 31, attention=1, feed_input=1, D=3)
    w = synth.make_weights(cfg, seed=3, scale=0.3)
    m = oracle.OracleModel(cfg, w)
    src, tin, tout = synth.make_s2s_batch(29, 31, 4, 3, 10, 3, 8, seed=9)
    full = m.score_batch(src, tin, tout)
    for b in range(4):
        s = src[:, b][src[:, b] != -1].reshape(-1, 1)
        n = int((tin[:, b] != -1).sum())
        one = m.score_batch(s, tin[:n, b:b + 1], tout[:n, b:b + 1])
        helpers.assert_logp_close(full[:n, b], one[:, 0], rtol=1e-6, atol=1e-6)


def test_synth_generators_are_deterministic():
    cfg = synth.make_cfg(1, 8, 11, 13, attention=2, feed_input=1)
    a = synth.make_weights(cfg, seed=5)
    b = synth.make_weights(cfg, seed=5)
    assert all(np.array_equal(x, y) for x, y in zip(a, b))
    assert len(a) == len(synth.tensor_spec(cfg))
    src, tin, tout = synth.make_s2s_batch(11, 13, 6, 2, 7, 2, 6, seed=1)
    assert src.shape[1] == 6 and tin.shape == tout.shape
    for bb in range(6):
        col = src[:, bb]
        n = (col != -1).sum()
        assert np.all(col[:len(col) - n] == -1) and np.all(col[len(col) - n:] != -1)  # left padded
        t = (tin[:, bb] != -1).sum()
        assert tin[0, bb] == 0 and tout[t - 1, bb] == 1 and np.all(tin[t:, bb] == -1)
    r = synth.to_bf16_f32(np.array([1.0, 1.00390625, 3.14159], dtype=np.float32))
    assert r[0] == 1.0 and (r.view(np.uint32) & 0xFFFF == 0).all()


def test_model_file_writer_layout(tmp_path):
    from zoph_rnn_b200.model_file import write_model_nn
    cfg = synth.make_cfg(1, 3, 4, 5)
    w = synth.make_weights(cfg, seed=1)
    p = tmp_path / "model.nn"
    write_model_nn(p, cfg, w)
    lines = p.read_text().split("\n")
    assert lines[0].split()[:4] == ["1", "3", "5", "4"]
    assert lines[1].startswith("===")
    # first matrix (W_hi of the source layer, 3x3) starts after header, 2 vocab sections and 3 separators
    start = 1 + 1 + 4 + 1 + 5 + 1
    first = np.array([[float(v) for v in lines[start + r].split()] for r in range(3)], dtype=np.float32)
    np.testing.assert_allclose(first, w[0].reshape(3, 3).T, rtol=1e-6)
    assert lines[start + 3] == ""


def test_library_exports_every_declared_symbol():
    """The C-ABI library loads without a GPU and exports everything include/zrnn.h and include/zrnn_debug.h declare."""
    from zoph_rnn_b200 import _lib
    hdr = open(os.path.join(ROOT, "include", "zrnn.h")).read() + open(os.path.join(ROOT, "include", "zrnn_debug.h")).read()
    declared = set(re.findall(r"\b(zrnn_[a-z0-9_]+)\s*\(", hdr))
    assert declared, "no declarations parsed"
    L = ctypes.CDLL(_lib.LIB_PATH)
    for name in sorted(declared):
        assert hasattr(L, name), f"{name} declared in include/ but not exported"
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)
    assert _lib.lib().zrnn_built_for_sm() == 100


def test_argument_errors_without_gpu():
    """Bad arguments and a missing device are reported as status codes, never as a crash or exit."""
    from zoph_rnn_b200 import _lib
    L = _lib.lib()
    h = ctypes.c_void_p()
    assert L.zrnn_hh_create(0, 0, ctypes.byref(h)) == _lib.E_ARG
    assert b"H must be positive" in L.zrnn_last_error()
    assert L.zrnn_softmax_create(10, 4, 0, 5, 3, ctypes.byref(h)) == _lib.E_ARG
    assert L.zrnn_att_create(8, 40, 1, 0, ctypes.byref(h)) == _lib.E_ARG
    c = _lib.ModelConfig(1, 8, 0, 10, 1, 1, 0, 10, 0)  # language model with attention: rejected
    assert L.zrnn_model_create(ctypes.byref(c), ctypes.byref(h)) == _lib.E_ARG
    assert L.zrnn_model_load_file(b"/nonexistent/model.nn", 1, 10, 0, ctypes.byref(h)) == _lib.E_IO
    assert L.zrnn_status_string(_lib.E_IO) == b"weight file error"
    import torch
    if not torch.cuda.is_available():
        assert L.zrnn_hh_create(8, 0, ctypes.byref(h)) == _lib.E_CUDA  # no CPU fallback
