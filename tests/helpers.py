"""Shared helpers for the parity tests."""
import glob
import os

import numpy as np

from zoph_rnn_b200 import synth

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

# fp32 path: per-token log-probs within 1e-5 relative of the oracle (plus a tiny absolute floor for
# log-probs near zero)
LOGP_RTOL = 1e-5
LOGP_ATOL = 2e-6


def golden_cases():
    return sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLDEN_DIR, "*.npz")))


def load_golden(name):
    g = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    cfg = {k: int(v) for k, v in zip(synth.CFG_KEYS, g["cfg"])}
    w = synth.make_weights(cfg, seed=int(g["seed"]), scale=float(g["scale"]))
    return cfg, w, g


def split_sources(flat, lens):
    out, p = [], 0
    for n in lens:
        out.append(np.asarray(flat[p:p + n], dtype=np.int32))
        p += int(n)
    return out


def assert_logp_close(got, want, rtol=LOGP_RTOL, atol=LOGP_ATOL):
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    err = np.abs(got - want)
    tol = atol + rtol * np.abs(want)
    bad = err > tol
    assert not bad.any(), f"max rel err {(err / np.maximum(np.abs(want), 1e-12)).max():.3e}, {bad.sum()} of {bad.size} out of tolerance"
