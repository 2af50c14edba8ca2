"""Front end: option handling and the integer files it prepares, checked on the CPU against the plain-Python
restatement of the reference's input_file_prep (oracle/textprep.py).  No device is touched (--prep-only)."""
import glob
import os

import numpy as np
import pytest

from oracle import textprep
from zoph_rnn_b200 import api, synth
from tests.helpers import make_text_fixture, run_cli

S2S = dict(num_layers=2, H=32, V_src=40, V_tgt=50, lm=False, attention=1, feed_input=1, D=10)
LM = dict(num_layers=1, H=32, V_src=0, V_tgt=50, lm=True, attention=0, feed_input=0, D=10)


def tmp_file(tmp_path, name):
    hits = glob.glob(os.path.join(str(tmp_path), "zoph_tmp_*", name))
    assert len(hits) == 1, hits
    return open(hits[0]).read()


def test_prep_force_decode_seq2seq(tmp_path):
    cfg = synth.make_cfg(**S2S)
    model, sp, tp, _ = make_text_fixture(str(tmp_path), cfg, 37, seed=5)
    rc, out = run_cli(["-f", sp, tp, model, "out.txt", "-L", "14", "--prep-only"], tmp_path)
    assert rc == 0, out
    got = tmp_file(tmp_path, "validation.txt")
    # sequence-to-sequence force-decode always prepares with minibatch 1 (src/main.cu:1160)
    want = textprep.integerize_nonlm(model, sp, tp, 14, 1)
    assert got == want
    assert "-2" in got and got.count("\n") % 4 == 0


@pytest.mark.parametrize("minibatch", [1, 4, 8])
def test_prep_force_decode_sequence(tmp_path, minibatch):
    cfg = synth.make_cfg(**LM)
    model, _, tp, _ = make_text_fixture(str(tmp_path), cfg, 95, seed=6)
    rc, out = run_cli(["-s", "-f", tp, model, "out.txt", "-L", "13", "-m", minibatch, "--prep-only"], tmp_path)
    assert rc == 0, out
    got = tmp_file(tmp_path, "validation.txt")
    assert got == textprep.integerize_lm(model, tp, 13, minibatch)
    assert (got.count("\n") // 4) % minibatch == 0  # the last minibatch is completed with -1 rows


def test_prep_decode(tmp_path):
    cfg = synth.make_cfg(**S2S)
    model, sp, _, _ = make_text_fixture(str(tmp_path), cfg, 21, seed=7)
    rc, out = run_cli(["-k", "3", model, "kbest.txt", "--decode-main-data-files", sp, "-L", "12", "--prep-only"], tmp_path)
    assert rc == 0, out
    want, sents = textprep.integerize_kbest(model, sp, 12)
    assert tmp_file(tmp_path, "kbest_tmp_0") == want
    assert 0 < len(sents) < 21  # some lines fall to the length cut-off


@pytest.mark.parametrize("args,msg", [
    (["-t", "a", "b", "m.nn"], "belongs to training"),
    (["--fsa", "x.fsa", "-k", "1", "m.nn", "o"], "outside this program"),
    (["-f", "a", "b"], "four arguements"),
    (["-s", "-f", "a", "b"], "three arguements"),
    (["--no-such-flag"], "unrecognised option"),
    (["-k", "1", "m.nn", "o"], "--decode-main-data-files"),
    (["-k", "1", "m1.nn", "m2.nn", "o", "--decode-main-data-files", "a"], "same number of inputs"),
    (["-k", "1", "m.nn", "o", "--decode-main-data-files", "a", "--dec-ratio", "0.5"], "only two inputs"),
    (["-k", "1", "m.nn", "o", "--decode-main-data-files", "a", "--dec-ratio", "1.5", "0.5"], "min decoding ratio"),
    (["-k", "1", "m.nn", "o", "--decode-main-data-files", "a", "-b", "0"], "beam size"),
    (["-k", "1", "m.nn", "o", "--decode-main-data-files", "a", "-p", "-1"], "penalty"),
    (["-b", "5"], "nothing to do"),
])
def test_option_errors(tmp_path, args, msg):
    rc, out = run_cli(args, tmp_path)
    assert rc != 0
    assert msg in out, out


def test_model_kind_must_match_sequence_flag(tmp_path):
    cfg = synth.make_cfg(**LM)
    model, _, tp, _ = make_text_fixture(str(tmp_path), cfg, 5, seed=8)
    rc, out = run_cli(["-f", tp, tp + "x", model, "out.txt", "--prep-only"], tmp_path)
    assert rc != 0 and "--sequence" in out


def test_no_device_fails_loudly(tmp_path):
    """Without a CUDA device the front end must stop with an error, not fall back to anything."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    cfg = synth.make_cfg(**LM)
    model, _, tp, _ = make_text_fixture(str(tmp_path), cfg, 5, seed=9)
    rc, out = run_cli(["-s", "-f", tp, model, "out.txt"], tmp_path)
    assert rc != 0 and "ERROR" in out
    assert not os.path.exists(os.path.join(str(tmp_path), "out.txt"))


def test_model_file_host_parser(tmp_path):
    """The memory-mapped, threaded matrix parser returns exactly the float32 values that were written, for plain,
    scientific, signed-zero and very small / large tokens, and reports truncated files."""
    cfg = synth.make_cfg(**S2S)
    model, _, _, w = make_text_fixture(str(tmp_path), cfg, 1, seed=10)
    hdr, n_ints, n_src, n_tgt = api.read_model_file_header(model)
    assert hdr[:6] == [2, 32, 50, 40, 1, 1] and n_ints == 9 and (n_src, n_tgt) == (40, 50)
    spec = synth.tensor_spec(cfg)
    got = api.read_model_file(model, [(r, c) for _, r, c in spec])
    for g, t in zip(got, w):
        assert np.array_equal(g, np.asarray(t, dtype=np.float32).ravel())
    # a large matrix goes through the thread pool
    rng = np.random.default_rng(0)
    m = (rng.standard_normal((700, 300)) * 10.0 ** rng.integers(-30, 30, size=(700, 300))).astype(np.float32)
    m[0, :4] = [0.0, -0.0, 1e-45, 3.4e38]
    path = os.path.join(str(tmp_path), "big.nn")
    with open(path, "w") as f:
        f.write("1 300 700 0 0 0 0 0 0\n" + "=" * 40 + "\n0 <START>\n" + "=" * 40 + "\n")
        np.savetxt(f, m, fmt="%.9g")
        f.write("\n")
        np.savetxt(f, m[:3], fmt="%+.8e")
        f.write("\n")
    a, b = api.read_model_file(path, [(700, 300), (3, 300)])
    assert np.array_equal(a.reshape(300, 700).T.view(np.uint32), m.view(np.uint32))
    assert np.array_equal(b.reshape(300, 3).T, m[:3])
    with pytest.raises(api.ZrnnError):
        api.read_model_file(path, [(700, 300), (3, 300), (2, 2)])
    with pytest.raises(api.ZrnnError):
        api.read_model_file(path, [(700, 301)])


def test_prep_decode_legacy_model_prefix(tmp_path):
    """--legacy-model 1: every integer source line starts with id 0 (src/input_file_prep.h:3108-3110)."""
    cfg = synth.make_cfg(**S2S)
    model, sp, _, _ = make_text_fixture(str(tmp_path), cfg, 9, seed=11)
    rc, out = run_cli(["-k", "1", model, "kbest.txt", "--decode-main-data-files", sp, "--legacy-model", "1",
                       "--prep-only"], tmp_path)
    assert rc == 0, out
    want, sents = textprep.integerize_kbest(model, sp, 100, legacy=True)
    assert tmp_file(tmp_path, "kbest_tmp_0") == want
    assert all(s[0] == 0 for s in sents)


def test_prep_decode_ensemble_writes_one_file_per_model(tmp_path):
    d1, d2 = tmp_path / "a", tmp_path / "b"
    d1.mkdir(); d2.mkdir()
    cfg = synth.make_cfg(**S2S)
    m1, s1, _, _ = make_text_fixture(str(d1), cfg, 6, seed=12)
    m2, s2, _, _ = make_text_fixture(str(d2), cfg, 6, seed=13)
    rc, out = run_cli(["-k", "1", m1, m2, "kbest.txt", "--decode-main-data-files", s1, s2, "--prep-only"], tmp_path)
    assert rc == 0, out
    assert tmp_file(tmp_path, "kbest_tmp_0") == textprep.integerize_kbest(m1, s1, 100)[0]
    assert tmp_file(tmp_path, "kbest_tmp_1") == textprep.integerize_kbest(m2, s2, 100)[0]
