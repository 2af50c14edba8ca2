"""World-size-2 gloo tests of the multi-GPU host logic on CPU.  The CUDA arithmetic is replaced by a stand-in built on
the CPU oracle; what is tested is the sharding, ordering and combination logic in zoph_rnn_b200/sharded.py."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from zoph_rnn_b200 import sharded, synth


def test_shard_bounds_cover_everything():
    for n in (1, 7, 128, 200000):
        for w in (1, 2, 3, 8):
            b = sharded.shard_bounds(n, w)
            assert b[0][0] == 0 and b[-1][1] == n
            assert all(b[i][1] == b[i + 1][0] for i in range(w - 1))
            sizes = [hi - lo for lo, hi in b]
            assert max(sizes) - min(sizes) <= 1


class OracleEngine:
    """CPU stand-in for CudaEngine: recurrent stack by the oracle, shard partials in NumPy."""

    def __init__(self, cfg, weights, rank, world):
        from oracle import oracle_lib
        self.cfg = cfg
        self.om = oracle_lib.OracleModel(cfg, weights)
        self.lo, self.hi = sharded.shard_bounds(cfg["V_tgt"], world)[rank]
        V, H = cfg["V_tgt"], cfg["H"]
        self.D = np.asarray(weights[-2], dtype=np.float64).reshape(H, V).T[self.lo:self.hi]   # rows of this shard
        self.b = np.asarray(weights[-1], dtype=np.float64)[self.lo:self.hi]

    def forward_states(self, src, tin):
        T, Bl = tin.shape
        dummy_out = np.where(tin == -1, -1, 1).astype(np.int32)
        _, top = self.om.score_batch(src, tin, dummy_out, want_top=True)
        return torch.as_tensor(top.reshape(T * Bl, self.cfg["H"]))

    def partials(self, h_all, targets):
        z = h_all.numpy().astype(np.float64) @ self.D.T + self.b
        mx = z.max(axis=1)
        sm = np.exp(z - mx[:, None]).sum(axis=1)
        t = targets.numpy()
        inside = (t >= self.lo) & (t < self.hi)
        tg = np.where(inside, z[np.arange(len(t)), np.clip(t - self.lo, 0, self.hi - self.lo - 1)], 0.0)
        return (torch.as_tensor(mx.astype(np.float32)), torch.as_tensor(sm.astype(np.float32)),
                torch.as_tensor(tg.astype(np.float32)))

    def combine(self, mx, sm, tg, mask):
        mx, sm, tg = mx.double(), sm.double(), tg.double()
        m = mx.max(dim=0).values
        s = (sm * torch.exp(mx - m)).sum(dim=0)
        return ((tg.sum(dim=0) - m - torch.log(s)) * mask.double()).float()

    def to_device(self, a):
        return torch.as_tensor(a)


def _worker(rank, world, port, cfg, seed, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        w = synth.make_weights(cfg, seed=seed, scale=0.3)
        src, tin, tout = synth.make_s2s_batch(cfg["V_src"], cfg["V_tgt"], 5, 3, 8, 3, 7, seed=seed)
        scorer = sharded.VocabShardedScorer(OracleEngine(cfg, w, rank, world), rank, world)
        lp = scorer.score(src, tin, tout)
        np.save(os.path.join(out_dir, f"lp{rank}.npy"), lp)
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world", [2, 3])
def test_vocab_sharded_scoring_matches_single_process(tmp_path, world):
    from oracle import oracle_lib
    cfg = synth.make_cfg(2, 12, 21, 23, attention=2, feed_input=1)
    seed = 5
    mp.spawn(_worker, args=(world, _free_port(), cfg, seed, str(tmp_path)), nprocs=world, join=True)
    w = synth.make_weights(cfg, seed=seed, scale=0.3)
    src, tin, tout = synth.make_s2s_batch(cfg["V_src"], cfg["V_tgt"], 5, 3, 8, 3, 7, seed=seed)
    want = oracle_lib.OracleModel(cfg, w).score_batch(src, tin, tout)
    for r in range(world):
        got = np.load(tmp_path / f"lp{r}.npy")
        np.testing.assert_allclose(got, want, rtol=2e-5, atol=2e-5)


def _shard_topk(z, lo, k):
    """What zrnn_softmax_topk_shard reports for the rows z [N, rows] of one shard (NumPy)."""
    N, rows = z.shape
    m = z.max(axis=1)
    lse = m + np.log(np.exp(z - m[:, None]).sum(axis=1))
    order = np.argsort(-z, axis=1, kind="stable")[:, :k]          # stable: ties to the lower row
    val = np.take_along_axis(z, order, axis=1) - lse[:, None]
    idx = order.astype(np.int32)
    if rows < k:
        val = np.concatenate([val, np.full((N, k - rows), -np.inf)], axis=1)
        idx = np.concatenate([idx, np.full((N, k - rows), -1, np.int32)], axis=1)
    eos = z[:, 1 - lo] - lse if lo <= 1 < lo + rows else np.full(N, -np.inf)
    return val.astype(np.float32), idx, lse.astype(np.float32), eos.astype(np.float32)


def _topk_worker(rank, world, port, V, H, N, k, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(3)
        D = rng.standard_normal((V, H))
        b = rng.standard_normal(V) * 0.1
        h = rng.standard_normal((N, H))
        bounds = sharded.shard_bounds(V, world)
        lo, hi = bounds[rank]
        val, idx, lse, eos = _shard_topk(h @ D[lo:hi].T + b[lo:hi], lo, k)
        # the library's wire format: one buffer of [N*k val | N*k idx | N lse | N eos] 4-byte words per rank
        mine = torch.as_tensor(np.concatenate([val.reshape(-1).view(np.int32), idx.reshape(-1), lse.view(np.int32),
                                               eos.view(np.int32)]))
        got = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(got, mine)
        words = np.stack([g.numpy() for g in got])
        vals = words[:, :N * k].view(np.float32).reshape(world, N, k)
        idxs = words[:, N * k:2 * N * k].reshape(world, N, k)
        lses = words[:, 2 * N * k:2 * N * k + N].view(np.float32)
        eoss = words[:, 2 * N * k + N:].view(np.float32)
        v, i, e = sharded.merge_topk_host(vals, idxs, lses, eoss, [a for a, _ in bounds], k)
        np.savez(os.path.join(out_dir, f"topk{rank}.npz"), v=v, i=i, e=e)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,V,k", [(2, 301, 13), (3, 40, 16)])
def test_sharded_topk_merge_matches_the_whole_vocabulary(tmp_path, world, V, k):
    """Per-shard top-k + all-gather + merge over gloo ranks equals the top-k of the whole softmax; with V = 40 over 3
    ranks every shard holds fewer rows than k."""
    H, N = 16, 9
    mp.spawn(_topk_worker, args=(world, _free_port(), V, H, N, k, str(tmp_path)), nprocs=world, join=True)
    rng = np.random.default_rng(3)
    D = rng.standard_normal((V, H))
    b = rng.standard_normal(V) * 0.1
    h = rng.standard_normal((N, H))
    z = h @ D.T + b
    logp = z - (z.max(axis=1, keepdims=True) + np.log(np.exp(z - z.max(axis=1, keepdims=True)).sum(axis=1, keepdims=True)))
    order = np.argsort(-logp, axis=1, kind="stable")[:, :k]
    for r in range(world):
        got = np.load(tmp_path / f"topk{r}.npz")
        np.testing.assert_array_equal(got["i"], order)
        np.testing.assert_allclose(got["v"], np.take_along_axis(logp, order, axis=1), rtol=1e-5, atol=1e-5)
        np.testing.assert_allclose(got["e"], logp[:, 1], rtol=1e-5, atol=1e-5)
