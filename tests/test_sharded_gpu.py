"""Vocabulary-sharded decoding and scoring behind the C ABI: per-shard top-k + merge against the unsharded top-k and
the oracle, the communicator with one rank, and (where the box has two GPUs) two ranks over NCCL."""
import os
import subprocess
import sys

import numpy as np
import pytest

from tests import helpers
from zoph_rnn_b200 import synth

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def api():
    from zoph_rnn_b200 import api as a
    return a


def dev(a):
    import torch
    return torch.as_tensor(a).cuda()


def build_model(api, cfg, w, dtype, shard=None):
    m = api.neuralMT_model(cfg, dtype=dtype, shard=shard)
    m.load_weights(w)
    return m


@pytest.mark.parametrize("dtype", [3, 0, 1])
@pytest.mark.parametrize("G", [2, 3, 8])
@pytest.mark.parametrize("V,H,N,k", [(1003, 64, 37, 13), (20011, 128, 130, 16), (50, 64, 5, 12),
                                     (5003, 64, 20, 33)])
def test_topk_shards_merge_to_the_unsharded_topk(api, oracle, G, dtype, V, H, N, k):
    """G shards on one GPU: zrnn_softmax_topk_shard per shard + zrnn_topk_merge against zrnn_softmax_topk of the whole
    layer (same word ids wherever the neighbours are no near-tie; values to fp32 rounding of the normaliser) and the
    oracle's distribution."""
    import torch
    rng = np.random.default_rng(G * 1000 + V)
    D = (rng.standard_normal(V * H) / np.sqrt(H)).astype(np.float32)
    b = (rng.standard_normal(V) * 0.1).astype(np.float32)
    h = (rng.standard_normal(H * N) * 2).astype(np.float32)
    full = api.softmax_layer(V, H, dtype=dtype)
    full.load_weights(D, b)
    wv, wi, we = (t.cpu().numpy() for t in full.topk(dev(h), k))
    vals, idxs, lses, eoss, los = [], [], [], [], []
    for g in range(G):
        lo, hi = api.shard_range(V, G, g)
        sm = api.softmax_layer(V, H, dtype=dtype, shard_lo=lo, shard_hi=hi)
        sm.load_weights(D, b)
        v, i, l, e = sm.topk_shard(dev(h), k)
        if not (lo <= 1 < hi):
            assert torch.isinf(e).all() and (e < 0).all()
        n_rows = hi - lo
        assert ((i >= 0).sum(dim=1) == min(k, n_rows)).all(), "a shard reports min(k, its rows) candidates"
        assert (i < n_rows).all()
        vals.append(v); idxs.append(i); lses.append(l); eoss.append(e); los.append(lo)
    gv, gi, ge = api.softmax_layer.merge_topk(torch.stack(vals), torch.stack(idxs), torch.stack(lses),
                                              torch.stack(eoss), los)
    torch.cuda.synchronize()
    assert api.lib().zrnn_tc_error() == 0
    gv, gi, ge = gv.cpu().numpy(), gi.cpu().numpy(), ge.cpu().numpy()
    tol = dict(rtol=2e-5, atol=2e-5) if dtype in (0, 3) else dict(rtol=2e-2, atol=2e-2)
    np.testing.assert_allclose(gv, wv, **tol)
    np.testing.assert_allclose(ge, we, **tol)
    # a row may differ only where two neighbouring values are within the tolerance of each other
    gap = np.abs(np.diff(wv, axis=1))
    clear = np.ones_like(wi, dtype=bool)
    thr = 1e-4 if dtype in (0, 3) else 5e-2
    clear[:, :-1] &= gap > thr
    clear[:, 1:] &= gap > thr
    clear[:, -1] = False  # the (k+1)-th value is not known here
    assert (gi[clear] == wi[clear]).all()
    assert (np.diff(gv, axis=1) <= 0).all(), "sorted descending"
    # and the host statement of the merge agrees bit for bit on the ids
    from zoph_rnn_b200 import sharded
    hv, hi_, he = sharded.merge_topk_host(torch.stack(vals).cpu().numpy(), torch.stack(idxs).cpu().numpy(),
                                          torch.stack(lses).cpu().numpy(), torch.stack(eoss).cpu().numpy(), los, k)
    np.testing.assert_array_equal(hi_, gi)
    np.testing.assert_allclose(hv, gv, rtol=1e-6, atol=1e-6)
    np.testing.assert_allclose(he, ge, rtol=1e-6, atol=1e-6)
    if dtype == 3:
        p = oracle.softmax_dist(V, H, N, D, b, h).reshape(N, V)
        np.testing.assert_allclose(np.exp(gv.astype(np.float64)), np.take_along_axis(p, gi.astype(np.int64), axis=1),
                                   rtol=1e-4, atol=1e-9)


def test_topk_merge_ties_go_to_the_lower_word_id(api):
    import torch
    G, N, k = 3, 2, 4
    val = torch.full((G, N, k), -1.5, device="cuda")
    idx = torch.tensor([[[0, 1, 2, 3]] * N] * G, dtype=torch.int32, device="cuda")
    lse = torch.zeros(G, N, device="cuda")
    eos = torch.full((G, N), float("-inf"), device="cuda")
    eos[1] = -2.0
    gv, gi, ge = api.softmax_layer.merge_topk(val, idx, lse, eos, [100, 0, 50])
    assert gi.cpu().tolist() == [[0, 1, 2, 3]] * N  # shard 1 holds the lowest ids
    np.testing.assert_allclose(gv.cpu().numpy(), -1.5 - np.log(3.0), rtol=1e-6)
    np.testing.assert_allclose(ge.cpu().numpy(), -2.0 - np.log(3.0), rtol=1e-6)


def test_sharded_calls_check_their_arguments(api):
    import torch
    cfg = synth.make_cfg(1, 64, 50, 60, attention=0, feed_input=0)
    w = synth.make_weights(cfg, seed=1, scale=0.1)
    comm = api.Communicator(None, 0, 1)
    plain = build_model(api, cfg, w, 3)
    sharded_m = build_model(api, cfg, w, 3, shard=(0, 30))  # not the range of rank 0 of 1
    src, tin, tout = synth.make_s2s_batch(50, 60, 3, 2, 5, 4, 4, seed=3)
    got, _ = plain.get_error_sharded(comm, src, tin, tout)  # one rank holding the whole vocabulary: allowed
    np.testing.assert_allclose(got, plain.get_error(src, tin, tout)[0], rtol=1e-6, atol=1e-6)
    with pytest.raises(api.ZrnnError) as e:
        sharded_m.get_error_sharded(comm, src, tin, tout)
    assert e.value.status == 1 and "share" in str(e.value)
    with pytest.raises(api.ZrnnError) as e:
        sharded_m.get_error(src, tin, tout)
    assert e.value.status == 1 and "sharded" in str(e.value)
    with pytest.raises(api.ZrnnError) as e:
        sharded_m.decode([np.array([3, 4], np.int32)], beam=3, longest_sent=10)
    assert e.value.status == 1
    with pytest.raises(api.ZrnnError) as e:
        api.Communicator(None, 0, 2)  # more than one rank needs the id
    assert e.value.status == 1
    with pytest.raises(api.ZrnnError):
        api.Communicator(None, 0, 9)
    import ctypes
    h = ctypes.c_void_p()
    assert api.lib().zrnn_comm_from_nccl(None, 0, 2, ctypes.byref(h)) == 1  # no communicator given


@pytest.mark.parametrize("dtype", [3, 5, 1])
def test_one_rank_communicator_equals_the_plain_calls(api, oracle, dtype):
    """world = 1: the sharded entry points take the whole vocabulary and must reproduce zrnn_score_batch and
    zrnn_beam_decode_batch (no NCCL involved)."""
    cfg = synth.make_cfg(2, 128, 300, 1000, attention=2, feed_input=1)
    w = synth.make_weights(cfg, seed=5, scale=0.2)
    comm = api.Communicator(None, 0, 1)
    plain = build_model(api, cfg, w, dtype)
    sh = build_model(api, cfg, w, dtype, shard=api.shard_range(1000, 1, 0))
    src, tin, tout = synth.make_s2s_batch(300, 1000, 7, 3, 9, 2, 8, seed=8)
    want, wt = plain.get_error(src, tin, tout)
    got, gt = sh.get_error_sharded(comm, src, tin, tout)
    if dtype == 1:
        np.testing.assert_allclose(got, want, rtol=1e-6, atol=1e-6)
    else:
        helpers.assert_logp_close(got, want)
        helpers.assert_logp_close(got, oracle.OracleModel(cfg, w).score_batch(src, tin, tout))
    assert abs(gt - wt) < 1e-3 * max(1.0, abs(wt))
    srcs = synth.make_decode_sources(300, 9, 3, 9, seed=2)
    kw = dict(beam=5, k_best=2, min_ratio=0.5, max_ratio=2.0, penalty=0.0, longest_sent=30)
    wi, wl, ws = plain.decode(srcs, **kw)
    gi, gl, gs = sh.decode_sharded(comm, srcs, **kw)
    np.testing.assert_array_equal(gl, wl)
    np.testing.assert_array_equal(gi, wi)
    np.testing.assert_allclose(gs, ws, rtol=1e-5, atol=1e-5)


def test_sharded_model_from_a_weight_file(api, tmp_path):
    """zrnn_model_load_file_sharded keeps the rank's rows of D; with one rank that is the whole model."""
    from zoph_rnn_b200.model_file import write_model_nn
    cfg = synth.make_cfg(2, 64, 40, 50, attention=1, feed_input=1, D=3)
    w = synth.make_weights(cfg, seed=2, scale=0.3)
    p = tmp_path / "model.nn"
    write_model_nn(p, cfg, w)
    comm = api.Communicator(None, 0, 1)
    m = api.neuralMT_model.from_file_sharded(p, comm, att_type=1, D=3, dtype=3)
    assert m.shard == (0, 50)
    src, tin, tout = synth.make_s2s_batch(40, 50, 5, 3, 9, 3, 8, seed=1)
    got, _ = m.get_error_sharded(comm, src, tin, tout)
    want, _ = build_model(api, cfg, w, 3).get_error(src, tin, tout)
    np.testing.assert_allclose(got, want, rtol=1e-6, atol=1e-6)
    with pytest.raises(api.ZrnnError):
        api.check(api.lib().zrnn_model_load_file_sharded(str(p).encode(), 1, 3, 3, 2, 5, None))


TWO_RANK_SCRIPT = r"""
import os, sys, time
import numpy as np
rank, world, idfile, outfile, dtype = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3], sys.argv[4], int(sys.argv[5])
sys.path.insert(0, os.getcwd())
import torch
torch.cuda.set_device(rank)
from zoph_rnn_b200 import api, synth, sharded
if rank == 0:
    uid = api.Communicator.unique_id()
    with open(idfile + ".tmp", "wb") as f:
        f.write(uid)
    os.replace(idfile + ".tmp", idfile)
else:
    t0 = time.time()
    while not os.path.exists(idfile):
        if time.time() - t0 > 120:
            sys.exit(3)
        time.sleep(0.05)
    uid = open(idfile, "rb").read()
comm = api.Communicator(uid, rank, world)
cfg = synth.make_cfg(2, 128, 300, 1001, attention=2, feed_input=1)
w = synth.make_weights(cfg, seed=5, scale=0.2)
m = sharded.ShardedModel(cfg, w, comm, dtype=dtype)
src, tin, tout = synth.make_s2s_batch(300, 1001, 7, 3, 9, 2, 8, seed=8)
lp, tot = m.score(src, tin, tout)
srcs = synth.make_decode_sources(300, 9, 3, 9, seed=2)
ids, ln, sc = m.decode(srcs, beam=5, k_best=2, min_ratio=0.5, max_ratio=2.0, penalty=0.0, longest_sent=30)
np.savez(outfile, lp=lp, tot=tot, ids=ids, ln=ln, sc=sc)
comm.close()
"""


@pytest.mark.parametrize("dtype", [3, 1])
def test_two_ranks_over_nccl(api, oracle, tmp_path, dtype):
    """Two processes, one GPU each, the library's own NCCL communicator: both ranks return the scores and hypotheses of
    the unsharded model."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "rank.py"
    script.write_text(TWO_RANK_SCRIPT)
    idfile = str(tmp_path / "nccl_id")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([sys.executable, str(script), str(r), "2", idfile, str(tmp_path / f"out{r}.npz"), str(dtype)],
                              cwd=ROOT, env=env) for r in range(2)]
    try:
        codes = [p.wait(timeout=300) for p in procs]
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
    assert codes == [0, 0]
    cfg = synth.make_cfg(2, 128, 300, 1001, attention=2, feed_input=1)
    w = synth.make_weights(cfg, seed=5, scale=0.2)
    plain = build_model(api, cfg, w, dtype)
    src, tin, tout = synth.make_s2s_batch(300, 1001, 7, 3, 9, 2, 8, seed=8)
    want, _ = plain.get_error(src, tin, tout)
    srcs = synth.make_decode_sources(300, 9, 3, 9, seed=2)
    wi, wl, ws = plain.decode(srcs, beam=5, k_best=2, min_ratio=0.5, max_ratio=2.0, penalty=0.0, longest_sent=30)
    outs = [np.load(tmp_path / f"out{r}.npz") for r in range(2)]
    np.testing.assert_array_equal(outs[0]["lp"], outs[1]["lp"])
    np.testing.assert_array_equal(outs[0]["ids"], outs[1]["ids"])
    for o in outs:
        if dtype == 3:
            helpers.assert_logp_close(o["lp"], want)
            helpers.assert_logp_close(o["lp"], oracle.OracleModel(cfg, w).score_batch(src, tin, tout))
            np.testing.assert_array_equal(o["ln"], wl)
            np.testing.assert_array_equal(o["ids"], wi)
            np.testing.assert_allclose(o["sc"], ws, rtol=1e-5, atol=1e-5)
        else:
            np.testing.assert_allclose(o["lp"], want, rtol=3e-2, atol=3e-2)
