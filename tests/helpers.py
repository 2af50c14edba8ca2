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


def make_text_fixture(dirpath, cfg, n_lines, seed, max_len=14, oov_rate=0.1, scale=None):
    """Writes a seeded model.nn plus source/target text files whose words come from the model's vocabulary (and some
    that do not).  Returns (model path, source path, target path, weights)."""
    from zoph_rnn_b200.model_file import default_vocab, write_model_nn
    w = synth.make_weights(cfg, seed=seed) if scale is None else synth.make_weights(cfg, seed=seed, scale=scale)
    model = os.path.join(dirpath, "model.nn")
    write_model_nn(model, cfg, w)
    srcw, tgtw = default_vocab(cfg)
    rng = np.random.default_rng(seed)
    sp, tp = os.path.join(dirpath, "src.txt"), os.path.join(dirpath, "tgt.txt")

    def sentence(words, first):
        n = int(rng.integers(1, max_len + 1))
        return " ".join("oov%d" % rng.integers(100) if rng.random() < oov_rate else words[int(rng.integers(first, len(words)))]
                        for _ in range(n))
    with open(sp, "w") as fs, open(tp, "w") as ft:
        for _ in range(n_lines):
            if not cfg["lm"]:
                fs.write(sentence(srcw, 1) + "\n")
            ft.write(sentence(tgtw, 3) + "\n")
    return model, sp, tp, w


CLI = os.path.join(os.path.dirname(GOLDEN_DIR), "..", "zoph_rnn_b200", "bin", "zoph_rnn")


def run_cli(args, cwd):
    """Runs the front end binary; returns (exit code, stdout + stderr)."""
    import subprocess
    from zoph_rnn_b200 import build
    build.build()
    p = subprocess.run([os.path.abspath(CLI)] + [str(a) for a in args], cwd=str(cwd), stdout=subprocess.PIPE,
                       stderr=subprocess.STDOUT, text=True, timeout=600)
    return p.returncode, p.stdout
