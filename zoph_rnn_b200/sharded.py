"""Multi-GPU host logic: sentence sharding (no collective) and vocabulary-sharded scoring / decoding.

The production path is ShardedModel below: the collective layer lives behind the C ABI (zrnn_comm_*,
zrnn_score_batch_sharded, zrnn_beam_decode_batch_sharded) and a host in any language drives it the same way.
VocabShardedScorer and merge_topk_host restate the same ordering and combination rules over torch.distributed, so
that they can be checked with gloo ranks on a machine without GPUs.

One process per GPU (torch.distributed).  Sentences are independent, so configs that fit one GPU shard the
minibatch by rank and never communicate.  A large-vocabulary model additionally shards the softmax matrix D by
rows: every rank runs the recurrent stack on its own sentences, the ranks all-gather the top-layer vectors
(H floats per token), each rank reduces its vocabulary rows to (max, sum exp, target logit) per token, and one
more all-gather of those three floats per token lets every rank finish log p = t - m - log(sum_g s_g e^(m_g - m)).
The engine object does the arithmetic (CUDA library in production, a CPU stand-in in the gloo tests).
"""
import numpy as np
import torch
import torch.distributed as dist


def shard_bounds(n, world):
    """Contiguous, near-equal [lo, hi) ranges of n items over `world` ranks."""
    # the same integer rule as zrnn_shard_range in the C ABI
    return [(n * r // world, n * (r + 1) // world) for r in range(world)]


def shard_columns(arr, rank, world):
    """Rank's sentences of a time-major [T, B] id array (columns = sentences)."""
    lo, hi = shard_bounds(arr.shape[1], world)[rank]
    return np.ascontiguousarray(arr[:, lo:hi])


class CudaEngine:
    """Arithmetic through libzrnn.so: a full recurrent stack plus this rank's rows of the softmax."""

    def __init__(self, cfg, weights, rank, world, dtype=0):
        from . import api
        self.api, self.cfg = api, cfg
        self.model = api.neuralMT_model(cfg, dtype=dtype)
        self.model.load_weights(weights)
        lo, hi = shard_bounds(cfg["V_tgt"], world)[rank]
        self.softmax = api.softmax_layer(cfg["V_tgt"], cfg["H"], dtype=dtype, shard_lo=lo, shard_hi=hi)
        self.softmax.load_weights(weights[-2], weights[-1])
        self.device = torch.device("cuda", torch.cuda.current_device())

    def forward_states(self, src, tin):
        """src [S,Bl] or None, tin [T,Bl] int32 arrays -> float32 tensor [T*Bl, H] on the device."""
        T, Bl = tin.shape
        d_src = torch.as_tensor(src).to(self.device) if src is not None else None
        d_tin = torch.as_tensor(tin).to(self.device)
        top = torch.empty(T * Bl, self.cfg["H"], dtype=torch.float32, device=self.device)
        self.model.forward_states_device(d_src, src.shape[0] if src is not None else 0, d_tin, T, Bl, top)
        return top

    def partials(self, h_all, targets):
        return self.softmax.partials(h_all.reshape(-1), targets)

    def combine(self, mx, sm, tg, mask):
        return self.api.softmax_layer.combine(mx, sm, tg, mask)

    def to_device(self, a):
        return torch.as_tensor(a).to(self.device)


class VocabShardedScorer:
    """Teacher-forced scoring of one minibatch by `world` ranks: sentences AND vocabulary rows are sharded."""

    def __init__(self, engine, rank, world):
        self.e, self.rank, self.world = engine, rank, world

    def score(self, src, tin, tout):
        """Full [T,B] inputs on every rank (each rank touches only its columns).  Returns log-probs [T,B]."""
        T, B = tin.shape
        bounds = shard_bounds(B, self.world)
        lo, hi = bounds[self.rank]
        mine = self.e.forward_states(None if src is None else np.ascontiguousarray(src[:, lo:hi]),
                                     np.ascontiguousarray(tin[:, lo:hi]))          # [T*Bl, H], column order t*Bl + b
        H = mine.shape[1]
        if self.world > 1:
            sizes = [T * (b - a) for a, b in bounds]
            pad = max(sizes)
            buf = torch.zeros(pad, H, dtype=mine.dtype, device=mine.device)
            buf[: mine.shape[0]] = mine
            gathered = [torch.empty_like(buf) for _ in range(self.world)]
            dist.all_gather(gathered, buf)
            parts = [g[:n] for g, n in zip(gathered, sizes)]
        else:
            parts = [mine]
        h_all = torch.cat(parts, dim=0).contiguous()                               # rank-major blocks of columns
        # targets / masks in the same rank-major column order
        order_t = np.concatenate([tout[:, a:b].reshape(-1) for a, b in bounds]).astype(np.int32)
        mask = (order_t != -1).astype(np.int32)
        tg_ids = np.where(order_t == -1, 0, order_t).astype(np.int32)
        d_tg, d_mask = self.e.to_device(tg_ids), self.e.to_device(mask)
        mx, sm, tg = self.e.partials(h_all, d_tg)
        if self.world > 1:
            mine3 = torch.stack([mx, sm, tg])                                      # [3, N]
            all3 = [torch.empty_like(mine3) for _ in range(self.world)]
            dist.all_gather(all3, mine3)
            mx, sm, tg = (torch.stack([a[i] for a in all3]).contiguous() for i in range(3))
        else:
            mx, sm, tg = mx[None], sm[None], tg[None]
        logp = self.e.combine(mx, sm, tg, d_mask).cpu().numpy()
        out = np.zeros((T, B), dtype=np.float32)
        pos = 0
        for a, b in bounds:
            n = T * (b - a)
            out[:, a:b] = logp[pos:pos + n].reshape(T, b - a)
            pos += n
        return out


def merge_topk_host(vals, idxs, lses, eoss, shard_lo, k):
    """NumPy statement of zrnn_topk_merge.  vals / idxs [G,N,k] (log-probabilities under each shard's own normaliser,
    row numbers inside the shard, -1 = no row), lses / eoss [G,N].  Returns (logp [N,k], word ids [N,k], eos [N])
    under the global normaliser; ties go to the lower word id."""
    vals = np.asarray(vals, dtype=np.float64)
    idxs = np.asarray(idxs)
    lses = np.asarray(lses, dtype=np.float64)
    eoss = np.asarray(eoss, dtype=np.float64)
    G, N, kk = vals.shape
    m = lses.max(axis=0)
    lse = m + np.log(np.exp(lses - m).sum(axis=0))
    glob = np.where(idxs >= 0, vals + lses[:, :, None] - lse[None, :, None], -np.inf)
    ids = np.where(idxs >= 0, idxs + np.asarray(shard_lo).reshape(G, 1, 1), np.iinfo(np.int32).max)
    glob = glob.transpose(1, 0, 2).reshape(N, G * kk)
    ids = ids.transpose(1, 0, 2).reshape(N, G * kk)
    out_v = np.empty((N, k), dtype=np.float32)
    out_i = np.empty((N, k), dtype=np.int32)
    for n in range(N):
        order = np.lexsort((ids[n], -glob[n]))[:k]
        out_v[n] = glob[n, order]
        out_i[n] = np.where(np.isfinite(glob[n, order]), ids[n, order], -1)
    with np.errstate(invalid="ignore"):
        e = np.where(np.isfinite(eoss), eoss + lses - lse[None, :], -np.inf).max(axis=0)
    return out_v, out_i, e.astype(np.float32)


class ShardedModel:
    """One rank of a vocabulary-sharded model: the recurrent stack and attention whole, rows
    [V r / world, V (r + 1) / world) of the softmax, and the library's communicator.  Every rank calls score() /
    decode() with the same arguments and gets the whole result."""

    def __init__(self, cfg, weights, comm, dtype=0):
        from . import api
        self.comm = comm
        self.model = api.neuralMT_model(cfg, dtype=dtype, shard=api.shard_range(cfg["V_tgt"], comm.world, comm.rank))
        self.model.load_weights(weights)

    def score(self, src, tin, tout):
        return self.model.get_error_sharded(self.comm, src, tin, tout)

    def decode(self, sources, **kw):
        return self.model.decode_sharded(self.comm, sources, **kw)
