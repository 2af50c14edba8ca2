"""Second, independent witness of the Zoph_RNN inference forward path, in float64 NumPy.

TEST INFRASTRUCTURE ONLY (same status as oracle/zoph_oracle.cpp): used by tests and by the
golden-vector generator to make sure a bug in the C++ oracle cannot silently become the spec.
It is written from the reference's math (cited below), not from the C++ oracle, and works in
float64 throughout, so agreement with the C++ oracle is expected to ~1e-6 relative, not bit-exact.

Conventions follow the reference: column-major H x B activations are represented here as
NumPy arrays of shape (B, H) (one row per sentence); token ids are time-major [T, B] with -1
padding; the source is reversed and left-padded, the target right-padded.
"""
import math

import numpy as np

ATT_NONE, ATT_LOCAL_P, ATT_GLOBAL_DOT = 0, 1, 2


def tensor_names(cfg):
    """Weight-file order (src/model.hpp:2172-2241, src/Input_To_Hidden_Layer.hpp:1104-1143,
    src/Hidden_To_Hidden_Layer.hpp:704-737, src/attention_layer.hpp:485-491, src/softmax.hpp:337-355)."""
    L, H = cfg["num_layers"], cfg["H"]
    out = []

    def lstm(prefix, emb_v, feed):
        for g in ("i", "f", "c", "o"):
            out.append((f"{prefix}.W_h{g}", H, H))
            out.append((f"{prefix}.b_{g}", H, 1))
        if emb_v:
            out.append((f"{prefix}.W", H, emb_v))
        for g in ("i", "f", "o", "c"):
            out.append((f"{prefix}.M_{g}", H, H))
        if feed:
            for g in ("i", "f", "o", "c"):
                out.append((f"{prefix}.Q_{g}", H, H))

    if not cfg["lm"]:
        for l in range(L):
            lstm(f"src{l}", cfg["V_src"] if l == 0 else 0, False)
    for l in range(L):
        lstm(f"tgt{l}", cfg["V_tgt"] if l == 0 else 0, l == 0 and cfg["feed_input"] and cfg["attention"])
        if cfg["attention"] and l == L - 1:
            out += [("att.W_a", H, H), ("att.W_p", H, H), ("att.v_p", 1, H), ("att.output_bias", H, 1),
                    ("att.W_c_p1", H, H), ("att.W_c_p2", H, H)]
    out += [("softmax.D", cfg["V_tgt"], H), ("softmax.b_d", cfg["V_tgt"], 1)]
    return out


def _as_dict(cfg, tensors):
    """tensors: list of column-major flat float arrays in file order -> {name: 2-D array (rows, cols)}"""
    d = {}
    for (name, r, c), t in zip(tensor_names(cfg), tensors):
        d[name] = np.asarray(t, dtype=np.float64).reshape(c, r).T  # column-major -> (rows, cols)
    return d


def _sigmoid(x):
    return 1.0 / (1.0 + np.exp(-x))


def _cell(w, p, x, h, c, htild, mask):
    """src/LSTM.hpp:133-399; x,h,c,htild: (B,H); mask: (B,)"""
    def pre(g):
        v = x @ w[f"{p}.M_{g}"].T + h @ w[f"{p}.W_h{g}"].T + w[f"{p}.b_{g}"][:, 0]
        if htild is not None:
            v = v + htild @ w[f"{p}.Q_{g}"].T
        return v
    i, f, o = _sigmoid(pre("i")), _sigmoid(pre("f")), _sigmoid(pre("o"))
    g = np.tanh(pre("c"))
    c2 = f * c + i * g
    h2 = o * np.tanh(c2)
    m = mask[:, None].astype(np.float64)
    return h2 * m, c2 * m


def _attention(cfg, w, h_t, mask, hs_all, lens, offs):
    """src/attention_node.hpp:73-394 (local-p) or the global-dot extension. hs_all: (S_max,B,H)."""
    B, H = h_t.shape
    ctx = np.zeros((B, H))
    D = cfg["D"]
    for b in range(B):
        if mask[b] != 1:
            continue
        Sb, ob = int(lens[b]), int(offs[b])
        if cfg["attention"] == ATT_LOCAL_P:
            s1 = float(w["att.v_p"][0] @ np.tanh(w["att.W_p"] @ h_t[b]))
            p = np.float32(Sb) * np.float32(_sigmoid(s1))          # float p_t as the kernel stores it
            ip = int(p)                                              # C cast, ck:1610-1611
            lo, hi = max(0, ip - D), min(Sb - 1, ip + D)
            q = w["att.W_a"].T @ h_t[b]
            pos = [j for j in range(lo, lo + 2 * D + 1) if j <= hi]
            if not pos:
                continue
            hs = np.stack([hs_all[Sb - 1 - j + ob, b] for j in pos])  # ck:1704
            e = hs @ q
            mx = max(0.0, float(e.max()))                            # max starts at 0, ck:1757
            a = np.exp(e - mx)
            s = a.sum()
            gauss = np.exp(-((float(p) - np.array(pos, dtype=np.float64)) ** 2) / (2.0 * (D * D / 4.0)))
            a = a / s * gauss if s != 0 else a                        # not renormalised, ck:1776-1783
            ctx[b] = a @ hs
        else:
            hs = np.stack([hs_all[Sb - 1 - j + ob, b] for j in range(Sb)])
            e = hs @ h_t[b]
            a = np.exp(e - e.max())
            a = a / a.sum()
            ctx[b] = a @ hs
    out = np.tanh(ctx @ w["att.W_c_p1"].T + h_t @ w["att.W_c_p2"].T + w["att.output_bias"][:, 0])
    return out * mask[:, None]


def _encode(cfg, w, src_ids):
    """src_ids [S,B] (-1 left padding). Returns final (h,c) per layer and top states (S,B,H)."""
    S, B = src_ids.shape
    L, H = cfg["num_layers"], cfg["H"]
    h = [np.zeros((B, H)) for _ in range(L)]
    c = [np.zeros((B, H)) for _ in range(L)]
    tops = np.zeros((S, B, H))
    for t in range(S):
        mask = (src_ids[t] != -1).astype(np.int64)
        ids = np.where(src_ids[t] == -1, 0, src_ids[t])
        x = w["src0.W"][:, ids].T
        for l in range(L):
            h[l], c[l] = _cell(w, f"src{l}", x, h[l], c[l], None, mask)
            x = h[l]
        tops[t] = h[L - 1]
    return h, c, tops


def score_batch(cfg, tensors, src_ids, tgt_in, tgt_out):
    """neuralMT_model::getError (src/model.hpp:1463-1802). Returns per-token ln p, shape [T,B]."""
    w = _as_dict(cfg, tensors)
    T, B = tgt_in.shape
    L, H = cfg["num_layers"], cfg["H"]
    if cfg["lm"]:
        h = [np.zeros((B, H)) for _ in range(L)]
        c = [np.zeros((B, H)) for _ in range(L)]
        tops, lens, offs = None, None, None
    else:
        h, c, tops = _encode(cfg, w, src_ids)
        lens = (src_ids != -1).sum(axis=0)
        offs = src_ids.shape[0] - lens
    htild = None
    out = np.zeros((T, B))
    for t in range(T):
        mask = (tgt_in[t] != -1).astype(np.int64)
        ids = np.where(tgt_in[t] == -1, 0, tgt_in[t])
        x = w["tgt0.W"][:, ids].T
        for l in range(L):
            feed = htild if (l == 0 and cfg["feed_input"] and cfg["attention"] and t != 0) else None
            h[l], c[l] = _cell(w, f"tgt{l}", x, h[l], c[l], feed, mask)
            x = h[l]
        top = h[L - 1]
        if cfg["attention"]:
            htild = _attention(cfg, w, h[L - 1], mask, tops, lens, offs)
            top = htild
        z = top @ w["softmax.D"].T + w["softmax.b_d"][:, 0]
        z = z - z.max(axis=1, keepdims=True)
        lp = z - np.log(np.exp(z).sum(axis=1, keepdims=True))
        y = np.where(tgt_out[t] == -1, 0, tgt_out[t])
        out[t] = np.where(tgt_out[t] != -1, lp[np.arange(B), y], 0.0)
    return out


def beam_decode_one(cfg, tensors, src, beam, k_best=1, min_ratio=0.5, max_ratio=1.5, penalty=0.0, longest_sent=100):
    """One sentence, reference style (src/ensemble_factory.hpp:583-765, src/decoder.h:1157-1315,
    672-688, 1386-1463). src: reversed source ids. Returns [(ids, score)] best first."""
    w = _as_dict(cfg, tensors)
    L, H, V = cfg["num_layers"], cfg["H"], cfg["V_tgt"]
    S = len(src)
    beam = min(beam, int(math.sqrt(V)))
    hS, cS, tops1 = _encode(cfg, w, np.asarray(src).reshape(S, 1))
    tops = np.repeat(tops1, beam, axis=1)
    lens, offs = np.full(beam, S), np.zeros(beam, dtype=np.int64)
    Lmax = longest_sent + 4
    sents = [[0] for _ in range(beam)]
    scores = np.zeros(beam)
    cur = [0] * beam
    hyps = []
    hp = [np.repeat(hS[l], beam, axis=0) for l in range(L)]
    cp = [np.repeat(cS[l], beam, axis=0) for l in range(L)]
    htild_feed = np.zeros((beam, H))
    ones = np.ones(beam, dtype=np.int64)

    def forward(idx):
        ids = [0 if i < 0 else i for i in cur]
        x = w["tgt0.W"][:, ids].T
        hn, cn = [], []
        for l in range(L):
            feed = htild_feed if (l == 0 and cfg["feed_input"] and cfg["attention"] and idx != 0) else None
            a, b = _cell(w, f"tgt{l}", x, hp[l], cp[l], feed, ones)
            hn.append(a); cn.append(b); x = a
        top, ht = hn[L - 1], None
        if cfg["attention"]:
            ht = _attention(cfg, w, hn[L - 1], ones, tops, lens, offs)
            top = ht
        z = top @ w["softmax.D"].T + w["softmax.b_d"][:, 0]
        z = z - z.max(axis=1, keepdims=True)
        return hn, cn, ht, z - np.log(np.exp(z).sum(axis=1, keepdims=True))

    max_steps = min(int(max_ratio * S), Lmax - 2)
    last = 0
    for step in range(max_steps):
        hn, cn, ht, logp = forward(step)
        cands = []
        for i in range(1 if step == 0 else beam):
            if cur[i] == -1:
                break
            top_idx = np.argsort(-logp[i], kind="stable")[: beam + 1]
            cands += [(logp[i, j] + scores[i], i, int(j)) for j in top_idx]
        cands.sort(key=lambda t: -t[0])
        new_sents, new_scores, new_cur, changes = [], [], [], []
        ci = 0
        while len(new_sents) < beam:
            if ci >= len(cands):
                new_sents.append(sents[0] + [0]); new_scores.append(0.0); new_cur.append(-1); changes.append(0)
                continue
            val, bi, j = cands[ci]; ci += 1
            if j == 0:
                continue
            if j == 1:
                hyps.append((sents[bi] + [1], val + penalty))
            else:
                new_sents.append(sents[bi] + [j]); new_scores.append(val + penalty); new_cur.append(j); changes.append(bi)
        sents, scores, cur = new_sents, np.array(new_scores), new_cur
        hp = [hn[l][changes] for l in range(L)]
        cp = [cn[l][changes] for l in range(L)]
        if cfg["feed_input"] and cfg["attention"]:
            htild_feed = ht[changes]
        last = step
    _, _, _, logp = forward(last + 1)
    for i in range(beam):
        if cur[i] == -1:
            continue
        hyps.append((sents[i] + [1], scores[i] + logp[i, 1] + penalty))
    keep = [h for h in hyps if np.float32(len(h[0])) / np.float32(S) > np.float32(min_ratio)]
    keep.sort(key=lambda t: -t[1])
    return keep[:k_best]
