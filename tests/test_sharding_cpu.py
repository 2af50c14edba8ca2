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
