"""Front end on a device: text in, the reference's output files out, checked against the CPU oracle run on the
integer files prepared by the plain-Python restatement of the reference's data preparation."""
import os

import numpy as np
import pytest

from oracle import textprep
from zoph_rnn_b200 import synth
from tests.helpers import make_text_fixture, run_cli

pytestmark = pytest.mark.gpu


def records(text):
    lines = text.split("\n")[:-1]
    return [[[int(x) for x in l.split()] for l in lines[i:i + 4]] for i in range(0, len(lines), 4)]


def oracle_unit_sums(om, recs, minibatch, lm):
    """Sum of ln p per minibatch of the integer file, one forward pass per minibatch as the reference does."""
    sums = []
    for u in range(0, len(recs), minibatch):
        grp = recs[u:u + minibatch]
        tin = np.array([r[2] for r in grp], dtype=np.int32).T
        tout = np.array([r[3] for r in grp], dtype=np.int32).T
        src = None if lm else np.array([r[0] for r in grp], dtype=np.int32).T
        sums.append(float(om.score_batch(src, np.ascontiguousarray(tin), np.ascontiguousarray(tout)).sum()))
    return sums


@pytest.mark.parametrize("dtype", ["f32", "f32-simt"])
@pytest.mark.parametrize("att", [1, 0])
def test_force_decode_seq2seq(tmp_path, oracle, att, dtype):
    cfg = synth.make_cfg(2, 128, 300, 400, attention=att, feed_input=att, D=4)
    model, sp, tp, w = make_text_fixture(str(tmp_path), cfg, 61, seed=12, max_len=17)
    rc, out = run_cli(["-f", sp, tp, model, "scores.txt", "-L", "18", "--attention-width", "4", "--dtype", dtype,
                       "--device-batch", "16", "--logfile", "log.txt"], tmp_path)
    assert rc == 0, out
    recs = records(textprep.integerize_nonlm(model, sp, tp, 18, 1))
    want = oracle_unit_sums(oracle.OracleModel(cfg, w), recs, 1, False)
    got = [float(x) for x in open(os.path.join(str(tmp_path), "scores.txt")).read().split()]
    assert len(got) == len(want) and len(got) > 20
    np.testing.assert_allclose(got, want, rtol=2e-5)  # 6 printed digits on top of the 1e-5 path tolerance
    words = sum(sum(1 for x in r[2] if x != -1) for r in recs)
    assert f"Total target words: {words}" in out
    ppl = float(out.split("Perplexity dev set: ")[1].split()[0])
    np.testing.assert_allclose(ppl, np.exp(-sum(want) / words), rtol=2e-5)
    assert "Perplexity dev set" in open(os.path.join(str(tmp_path), "log.txt")).read()
    assert not [d for d in os.listdir(str(tmp_path)) if d.startswith("zoph_tmp_")]  # tmp directory removed


@pytest.mark.parametrize("minibatch", [1, 4])
def test_force_decode_sequence(tmp_path, oracle, minibatch):
    cfg = synth.make_cfg(2, 128, 0, 400, lm=True)
    model, _, tp, w = make_text_fixture(str(tmp_path), cfg, 50, seed=13, max_len=17)
    rc, out = run_cli(["-s", "-f", tp, model, "scores.txt", "-L", "16", "-m", minibatch], tmp_path)
    assert rc == 0, out
    recs = records(textprep.integerize_lm(model, tp, 16, minibatch))
    want = oracle_unit_sums(oracle.OracleModel(cfg, w), recs, minibatch, True)
    got = [float(x) for x in open(os.path.join(str(tmp_path), "scores.txt")).read().split()]
    assert len(got) == len(want)
    np.testing.assert_allclose(got, want, rtol=2e-5)


@pytest.mark.parametrize("print_score", [0, 1])
def test_decode(tmp_path, oracle, print_score):
    cfg = synth.make_cfg(2, 64, 200, 300, attention=1, feed_input=1, D=3)
    model, sp, _, w = make_text_fixture(str(tmp_path), cfg, 24, seed=14, max_len=12, scale=0.25)
    rc, out = run_cli(["-k", "2", model, "kbest.txt", "--decode-main-data-files", sp, "-b", "6", "-L", "40",
                       "--attention-width", "3", "--dec-ratio", "0.5", "2.0", "-p", "0.1", "--print-score", print_score,
                       "--device-batch", "7"], tmp_path)
    assert rc == 0, out
    _, sents = textprep.integerize_kbest(model, sp, 40)
    ids, ln, sc = oracle.OracleModel(cfg, w).beam_decode([np.array(s, dtype=np.int32) for s in sents], beam=6, k_best=2,
                                                         min_ratio=0.5, max_ratio=2.0, penalty=0.1, longest_sent=40)
    hyps = [[(list(ids[s, h, :ln[s, h]]), float(sc[s, h])) for h in range(2) if ln[s, h] > 0] for s in range(len(sents))]
    got = open(os.path.join(str(tmp_path), "kbest.txt")).read()
    if not print_score:
        assert got == textprep.unint(model, textprep.format_kbest_ints(hyps, False))
    else:
        want = textprep.unint(model, textprep.format_kbest_ints(hyps, True)).split("\n")
        lines = got.split("\n")
        assert len(lines) == len(want)
        for g, x in zip(lines, want):
            if x.startswith("-Score: "):
                np.testing.assert_allclose(float(g[8:]), float(x[8:]), rtol=1e-4, atol=1e-4)
            else:
                assert g == x
    assert got.count("<START>") >= len(sents) and got.count("<EOF>") >= len(sents)


def test_decode_unk_replacement_file(tmp_path, oracle):
    """--UNK-decode: the alignment file lists, per hypothesis, the source position aligned to every <UNK>."""
    cfg = synth.make_cfg(2, 64, 200, 30, attention=1, feed_input=1, D=3)  # small target vocabulary: many <UNK>
    model, sp, _, w = make_text_fixture(str(tmp_path), cfg, 20, seed=15, max_len=12, scale=0.25)
    # make <UNK> (id 2) likely: raise its softmax bias
    from zoph_rnn_b200.model_file import write_model_nn
    w[-1] = np.array(w[-1], dtype=np.float32)
    w[-1][2] += 1.5
    write_model_nn(model, cfg, w)
    rc, out = run_cli(["-k", "2", model, "kbest.txt", "--decode-main-data-files", sp, "-b", "5", "-L", "40",
                       "--attention-width", "3", "--UNK-decode", "unk.txt"], tmp_path)
    assert rc == 0, out
    _, sents = textprep.integerize_kbest(model, sp, 40)
    ids, ln, sc, al = oracle.OracleModel(cfg, w).beam_decode([np.array(s, dtype=np.int32) for s in sents], beam=5,
                                                             k_best=2, longest_sent=40, want_align=True)
    hyps = [[(list(ids[s, h, :ln[s, h]]), list(al[s, h, :ln[s, h] + 1])) for h in range(2) if ln[s, h] > 0]
            for s in range(len(sents))]
    want_text = textprep.unint(model, textprep.format_kbest_ints([[(i, 0.0) for i, _ in sent] for sent in hyps], False))
    got_text = open(os.path.join(str(tmp_path), "kbest.txt")).read()
    got_unk = open(os.path.join(str(tmp_path), "unk.txt")).read()
    want_unk = textprep.format_unk_file(hyps)
    assert got_unk.count("\n") == want_unk.count("\n") == sum(len(s) for s in hyps)
    assert sum(len(l.split()) for l in want_unk.split("\n")) > 10  # the fixture does produce <UNK>s
    if got_text == want_text:  # same hypotheses: the alignments must match line by line (near-ties aside)
        g, x = got_unk.split("\n"), want_unk.split("\n")
        same = sum(a == b for a, b in zip(g, x))
        assert same >= 0.95 * len(x), (same, len(x))


def test_decode_ensemble_of_two_models(tmp_path, oracle):
    d1, d2 = tmp_path / "m1", tmp_path / "m2"
    d1.mkdir(); d2.mkdir()
    cfg_a = synth.make_cfg(2, 64, 200, 300, attention=1, feed_input=1, D=3)
    cfg_b = synth.make_cfg(1, 64, 120, 300, attention=0, feed_input=0)
    ma, sa, _, wa = make_text_fixture(str(d1), cfg_a, 15, seed=16, max_len=10, scale=0.25)
    mb, sb, _, wb = make_text_fixture(str(d2), cfg_b, 15, seed=17, max_len=10, scale=0.25)
    rc, out = run_cli(["-k", "1", ma, mb, "kbest.txt", "--decode-main-data-files", sa, sb, "-b", "5", "-L", "40",
                       "--attention-width", "3", "--device-batch", "4"], tmp_path)
    assert rc == 0, out
    _, xa = textprep.integerize_kbest(ma, sa, 40)
    _, xb = textprep.integerize_kbest(mb, sb, 40)
    ids, ln, sc = oracle.beam_decode_ensemble([oracle.OracleModel(cfg_a, wa), oracle.OracleModel(cfg_b, wb)],
                                              [[np.array(s, dtype=np.int32) for s in xa],
                                               [np.array(s, dtype=np.int32) for s in xb]], beam=5, k_best=1, longest_sent=40)
    hyps = [[(list(ids[s, 0, :ln[s, 0]]), float(sc[s, 0]))] if ln[s, 0] > 0 else [] for s in range(len(xa))]
    assert open(os.path.join(str(tmp_path), "kbest.txt")).read() == textprep.unint(ma, textprep.format_kbest_ints(hyps, False))


def _two_gpus():
    import torch
    return torch.cuda.device_count() >= 2


@pytest.mark.parametrize("devices", [["0", "0", "0"], ["0", "1", "1"]])
def test_multi_gpu_flag_shards_sentences(tmp_path, devices):
    """-M g0 g1 ... : repeated indices are one device (the reference's `-M 0 0 0`), every distinct device gets a worker
    process with a share of the device batches; the output files are byte-identical to the single-device run."""
    if len(set(devices)) > 1 and not _two_gpus():
        pytest.skip("needs two GPUs")
    cfg = synth.make_cfg(2, 64, 200, 300, attention=1, feed_input=1, D=3)
    model, sp, tp, w = make_text_fixture(str(tmp_path), cfg, 40, seed=21, max_len=12, scale=0.25)
    score_args = ["-f", sp, tp, model, None, "-L", "14", "--attention-width", "3", "--device-batch", "8"]
    dec_args = ["-k", "2", model, None, "--decode-main-data-files", sp, "-b", "5", "-L", "30", "--attention-width", "3",
                "--dec-ratio", "0.5", "2.0", "--print-score", "1", "--device-batch", "6", "--UNK-decode", None]
    outs = {}
    for tag, extra in (("one", []), ("many", ["-M"] + devices)):
        a = [f"scores_{tag}.txt" if x is None else x for x in score_args] + extra
        rc, out = run_cli(a, tmp_path)
        assert rc == 0, out
        if tag == "many" and len(set(devices)) > 1:
            assert "Sharding the sentences over 2 devices" in out
        ppl = out.split("Perplexity dev set: ")[1].split()[0]
        b = list(dec_args)
        b[3], b[-1] = f"kbest_{tag}.txt", f"unk_{tag}.txt"
        rc, out = run_cli(b + extra, tmp_path)
        assert rc == 0, out
        outs[tag] = (open(tmp_path / f"scores_{tag}.txt").read(), ppl, open(tmp_path / f"kbest_{tag}.txt").read(),
                     open(tmp_path / f"unk_{tag}.txt").read())
    assert outs["one"] == outs["many"]
    assert len(outs["one"][0].split()) == 40 or len(outs["one"][0].split()) > 20
    assert not [d for d in os.listdir(str(tmp_path)) if d.startswith("zoph_tmp_")]


def test_multi_gpu_flag_rejects_missing_devices(tmp_path):
    cfg = synth.make_cfg(1, 64, 50, 60, attention=0, feed_input=0)
    model, sp, tp, w = make_text_fixture(str(tmp_path), cfg, 5, seed=22, max_len=8)
    rc, out = run_cli(["-f", sp, tp, model, "s.txt", "-M", "0", "63"], tmp_path)
    assert rc != 0 and "only" in out and "visible" in out
