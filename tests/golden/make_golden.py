"""Generates the committed golden vectors (tests/golden/*.npz).

The reference ships no golden vectors for this path and cannot be built here, so the goldens are
produced by the float64 NumPy witness (oracle/ref_numpy.py) and cross-checked against the C++
oracle (oracle/zoph_oracle.cpp) before being written.  Weights are not stored: they are
regenerated from (cfg, seed) by zoph_rnn_b200.synth.make_weights.

Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle_lib as ol  # noqa: E402
from oracle import ref_numpy as rn  # noqa: E402
from zoph_rnn_b200 import synth  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))

CASES = {
    # name: (cfg, weight seed, weight scale, batch spec)
    "lm_2layer": (synth.make_cfg(2, 24, 0, 61, lm=1), 11, 0.3, dict(kind="lm", B=5, T=9)),
    "s2s_plain": (synth.make_cfg(2, 20, 43, 47), 12, 0.3, dict(kind="s2s", B=6, S=(3, 9), T=(3, 8))),
    "s2s_localp_feed": (synth.make_cfg(2, 32, 43, 47, attention=1, feed_input=1, D=3), 13, 0.3,
                        dict(kind="s2s", B=7, S=(4, 12), T=(3, 9))),
    "s2s_global_feed": (synth.make_cfg(3, 28, 43, 47, attention=2, feed_input=1), 14, 0.3,
                        dict(kind="s2s", B=6, S=(3, 10), T=(3, 8))),
    "s2s_localp_1layer": (synth.make_cfg(1, 17, 43, 47, attention=1, feed_input=0, D=2), 15, 0.3,
                          dict(kind="s2s", B=4, S=(5, 9), T=(4, 7))),
}
DECODE = dict(beam=5, k_best=3, min_ratio=0.5, max_ratio=1.5, penalty=0.0, longest_sent=30, n_sent=5, S=(3, 9))


def main():
    for name, (cfg, seed, scale, spec) in CASES.items():
        w = synth.make_weights(cfg, seed=seed, scale=scale)
        if spec["kind"] == "lm":
            src = None
            tin, tout = synth.make_lm_batch(cfg["V_tgt"], spec["B"], spec["T"], seed=seed)
        else:
            src, tin, tout = synth.make_s2s_batch(cfg["V_src"], cfg["V_tgt"], spec["B"], spec["S"][0], spec["S"][1],
                                                  spec["T"][0], spec["T"][1], seed=seed)
        lp = rn.score_batch(cfg, w, src, tin, tout)
        om = ol.OracleModel(cfg, w)
        lp_c = om.score_batch(src, tin, tout)
        err = np.abs(lp - lp_c).max()
        assert err < 5e-6, (name, err)
        out = dict(cfg=np.array([cfg[k] for k in synth.CFG_KEYS], dtype=np.int32), seed=seed, scale=scale,
                   tgt_in=tin, tgt_out=tout, logp=lp)
        if src is not None:
            out["src"] = src
            d = DECODE
            srcs = synth.make_decode_sources(cfg["V_src"], d["n_sent"], d["S"][0], d["S"][1], seed=seed + 100)
            ids, ln, sc = om.beam_decode(srcs, d["beam"], d["k_best"], d["min_ratio"], d["max_ratio"], d["penalty"],
                                         d["longest_sent"])
            for i, s in enumerate(srcs):  # the two witnesses must agree on every hypothesis
                r = rn.beam_decode_one(cfg, w, s, d["beam"], d["k_best"], d["min_ratio"], d["max_ratio"], d["penalty"],
                                       d["longest_sent"])
                for k in range(d["k_best"]):
                    got = list(ids[i, k, :ln[i, k]])
                    exp = r[k][0] if k < len(r) else []
                    assert got == exp, (name, i, k, got, exp)
                    if k < len(r):
                        assert abs(sc[i, k] - r[k][1]) < 1e-4, (name, i, k)
            out.update(dec_src=np.concatenate(srcs), dec_len=np.array([len(s) for s in srcs], dtype=np.int32),
                       dec_ids=ids, dec_hyp_len=ln, dec_score=sc)
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
        print(name, "ok; oracle-vs-witness max abs err", err)


if __name__ == "__main__":
    main()
