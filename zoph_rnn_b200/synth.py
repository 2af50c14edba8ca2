"""Seeded synthetic weights and token batches with the shapes and value distributions of the
five benchmark configurations.  No corpus or trained model ships with the reference, so every
parity test and benchmark run uses these generators; the same (seed, tensor index) always gives
the same values on any machine (counter-based Philox), so nothing has to be shipped as files.
"""
import math

import numpy as np

ATT_NONE, ATT_LOCAL_P, ATT_GLOBAL_DOT = 0, 1, 2
CFG_KEYS = ("num_layers", "H", "V_src", "V_tgt", "lm", "attention", "feed_input", "D")


def make_cfg(num_layers, H, V_src, V_tgt, lm=0, attention=ATT_NONE, feed_input=0, D=10):
    return dict(num_layers=num_layers, H=H, V_src=0 if lm else V_src, V_tgt=V_tgt, lm=int(lm), attention=int(attention),
                feed_input=int(feed_input and attention), D=D)


def tensor_spec(cfg):
    """(name, rows, cols) of every tensor in the order the reference's weight file stores them
    (src/model.hpp:2172-2241; per layer src/Input_To_Hidden_Layer.hpp:1104-1143 and
    src/Hidden_To_Hidden_Layer.hpp:704-737; attention src/attention_layer.hpp:485-491; softmax
    src/softmax.hpp:337-355)."""
    L, H = cfg["num_layers"], cfg["H"]
    out = []

    def lstm(prefix, emb_v, feed):
        for g in "ifco":
            out.append((f"{prefix}.W_h{g}", H, H))
            out.append((f"{prefix}.b_{g}", H, 1))
        if emb_v:
            out.append((f"{prefix}.W", H, emb_v))
        for g in "ifoc":
            out.append((f"{prefix}.M_{g}", H, H))
        if feed:
            for g in "ifoc":
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


def make_weights(cfg, seed=1234, dist="uniform", scale=0.1, round_bf16=False):
    """List of flat float32 arrays (column-major) in weight-file order.
    dist 'uniform' -> U[-scale, scale]; 'normal' -> N(0, scale)."""
    out = []
    for i, (_, r, c) in enumerate(tensor_spec(cfg)):
        g = np.random.Generator(np.random.Philox(key=[seed, i]))
        if dist == "uniform":
            a = g.random(r * c, dtype=np.float32)
            a *= np.float32(2 * scale)
            a -= np.float32(scale)
        else:
            a = g.standard_normal(r * c, dtype=np.float32)
            a *= np.float32(scale)
        if round_bf16:
            a = to_bf16_f32(a)
        out.append(a)
    return out


def to_bf16_f32(a):
    """Round float32 to the nearest bfloat16 (ties to even) and return it as float32."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return r.astype(np.uint32).view(np.float32)


def zipf_sampler(V, s, seed):
    """Token sampler with P(rank r) proportional to r^-s, ranks mapped to ids by a seeded permutation."""
    g = np.random.Generator(np.random.Philox(key=[seed, 7777]))
    p = np.arange(1, V + 1, dtype=np.float64) ** (-s)
    cdf = np.cumsum(p / p.sum())
    perm = g.permutation(V).astype(np.int32)

    def sample(gen, n):
        r = np.searchsorted(cdf, gen.random(n), side="right")
        return perm[np.minimum(r, V - 1)]
    return sample


def make_lm_batch(V, B, T, seed=1234, zipf_s=None):
    """Language-model batch: tgt_in[T,B] starts with <START>=0, tgt_out is tgt_in shifted by one."""
    g = np.random.Generator(np.random.Philox(key=[seed, 1]))
    if zipf_s:
        toks = zipf_sampler(V, zipf_s, seed)(g, B * (T + 1)).reshape(T + 1, B)
    else:
        toks = g.integers(0, V, size=(T + 1, B), dtype=np.int32)
    toks = toks.astype(np.int32)
    tgt_in = toks[:-1].copy()
    tgt_in[0, :] = 0
    tgt_out = toks[1:].copy()
    return tgt_in, tgt_out


def make_s2s_batch(V_src, V_tgt, B, S_min, S_max, T_min, T_max, seed=1234, zipf_s=1.1):
    """Sequence-to-sequence batch in the reference's minibatch layout (src/fileHelper.h:367-518):
    src_ids [S_max,B] reversed and LEFT-padded with -1; tgt_in [T,B] = <START> y1..yn right-padded with -1;
    tgt_out [T,B] = y1..yn <EOF>(=1) right-padded with -1.  Target tokens avoid ids 0 and 1."""
    g = np.random.Generator(np.random.Philox(key=[seed, 2]))
    ssrc = zipf_sampler(V_src, zipf_s, seed + 1)
    stgt = zipf_sampler(V_tgt, zipf_s, seed + 2)
    s_len = g.integers(S_min, S_max + 1, size=B)
    t_len = g.integers(T_min, T_max + 1, size=B)  # includes the <START>/<EOF> position
    S, T = int(s_len.max()), int(t_len.max())
    src = np.full((S, B), -1, dtype=np.int32)
    tin = np.full((T, B), -1, dtype=np.int32)
    tout = np.full((T, B), -1, dtype=np.int32)
    for b in range(B):
        src[S - s_len[b]:, b] = ssrc(g, int(s_len[b]))
        y = stgt(g, int(t_len[b]) - 1)
        y = np.where(y < 2, y + 2, y)
        tin[0, b] = 0
        tin[1:t_len[b], b] = y
        tout[:t_len[b] - 1, b] = y
        tout[t_len[b] - 1, b] = 1
    return src, tin, tout


def make_decode_sources(V_src, n_sent, S_min, S_max, seed=1234, zipf_s=1.1):
    """List of reversed source id arrays, one per sentence (decode input format,
    src/file_helper_decoder.h:75-131: no padding)."""
    g = np.random.Generator(np.random.Philox(key=[seed, 3]))
    ssrc = zipf_sampler(V_src, zipf_s, seed + 1)
    lens = g.integers(S_min, S_max + 1, size=n_sent)
    return [ssrc(g, int(n)).astype(np.int32) for n in lens]


def beam_cap(beam, V):
    """The reference caps the beam at floor(sqrt(V)) (src/ensemble_factory.hpp:19-21)."""
    return min(beam, int(math.sqrt(V)))
