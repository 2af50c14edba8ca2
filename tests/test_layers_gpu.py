"""GPU parity tests, layer by layer, through the C ABI against the CPU oracle."""
import numpy as np
import pytest

from tests import helpers
from zoph_rnn_b200 import synth

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def api():
    import torch
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    from zoph_rnn_b200 import api as a
    return a


# (dtype id, relative tolerance, absolute tolerance): exact engines first, then the reduced-precision ones
# ZRNN_F32_SIMT, ZRNN_F32_3XTF32, ZRNN_F32_F16X2 (tensor-core accumulation truncates)
EXACT = [(3, 2e-5, 2e-6), (4, 6e-5, 3e-5), (5, 6e-5, 3e-5)]
LOOSE = [(1, 3e-2, 3e-2), (2, 1e-2, 1e-2)]       # ZRNN_BF16, ZRNN_TF32


def engines_for(H):
    out = [EXACT[0]]
    if H % 4 == 0:
        out += [EXACT[1], EXACT[2], LOOSE[1]]
    if H % 8 == 0:
        out.append(LOOSE[0])
    return out


def dev(a, dtype=None):
    import torch
    t = torch.as_tensor(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda()


def rand_lstm(rng, H, V, feed, scale=0.3):
    """17-slot weight list in file order (None where absent) + the dense list the layer loads."""
    w = [None] * 17
    for g in range(4):
        w[2 * g] = (rng.standard_normal(H * H) * scale).astype(np.float32)
        w[2 * g + 1] = (rng.standard_normal(H) * scale).astype(np.float32)
    if V:
        w[8] = (rng.standard_normal(H * V) * scale).astype(np.float32)
    for k in range(9, 13):
        w[k] = (rng.standard_normal(H * H) * scale).astype(np.float32)
    if feed:
        for k in range(13, 17):
            w[k] = (rng.standard_normal(H * H) * scale).astype(np.float32)
    return w, [t for t in w if t is not None]


def test_prep_vocab_indices(api):
    import torch
    raw = np.array([5, -1, 0, 7, -1, -1, 3], dtype=np.int32)
    ids, mask = api.prep_vocab_indices(dev(raw))
    torch.cuda.synchronize()
    assert ids.cpu().tolist() == [5, 0, 0, 7, 0, 0, 3]
    assert mask.cpu().tolist() == [1, 0, 1, 1, 0, 0, 1]


@pytest.mark.parametrize("H,V,n", [(1, 5, 3), (3, 33, 7), (32, 50, 64), (100, 1000, 280), (1000, 5000, 640), (2048, 300, 17)])
def test_gather_is_bit_exact(api, oracle, H, V, n):
    rng = np.random.default_rng(H * 7 + V)
    w, dense = rand_lstm(rng, H, V, False, scale=1.0) if H <= 100 else (None, None)
    if w is None:  # large H: only the embedding matters; keep the H x H matrices tiny by loading a thin layer
        W = rng.standard_normal(H * V).astype(np.float32)
        z = np.zeros(H * H, dtype=np.float32)
        zb = np.zeros(H, dtype=np.float32)
        dense = [z, zb, z, zb, z, zb, z, zb, W, z, z, z, z]
    else:
        W = w[8]
    ids = rng.integers(0, V, size=n).astype(np.int32)
    ids[0] = V - 1
    ids[-1] = 0
    layer = api.Input_To_Hidden_Layer(H, V)
    layer.load_weights(dense)
    x = layer.gather(dev(ids)).cpu().numpy()
    want = oracle.gather(W, H, ids)
    assert np.array_equal(x.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("H,B,feed", [(1, 1, False), (3, 2, True), (32, 7, False), (33, 5, True), (100, 8, False),
                                       (100, 70, True), (256, 128, True), (1000, 12, False), (1000, 200, True),
                                       (264, 130, True)])
def test_lstm_cell_matches_oracle(api, oracle, H, B, feed):
    import torch
    rng = np.random.default_rng(H * 131 + B)
    V = 11
    scale = 0.5 / np.sqrt(H)
    w, dense = rand_lstm(rng, H, V, feed, scale=scale)
    ids = rng.integers(0, V, size=B).astype(np.int32)
    mask = (rng.random(B) > 0.25).astype(np.int32)
    mask[0] = 1
    h0 = rng.standard_normal(H * B).astype(np.float32) * 0.5
    c0 = rng.standard_normal(H * B).astype(np.float32) * 0.5
    ht = rng.standard_normal(H * B).astype(np.float32) * 0.5 if feed else None
    x = oracle.gather(w[8], H, ids)
    want_h, want_c = oracle.lstm_cell(H, B, w, x, h0, c0, ht, mask)
    want_h2, want_c2 = oracle.lstm_cell(H, B, w, h0, h0, c0, None, mask)
    for dtype, rtol, atol in engines_for(H):
        ih = api.Input_To_Hidden_Layer(H, V, feed_input=feed, dtype=dtype)
        ih.load_weights(dense)
        h, c = ih.forward_prop(dev(ids), dev(mask), dev(h0), dev(c0), dev(ht) if feed else None)
        torch.cuda.synchronize()
        assert api.lib().zrnn_tc_error() == 0
        np.testing.assert_allclose(h.cpu().numpy(), want_h, rtol=rtol, atol=atol, err_msg=f"dtype {dtype}")
        np.testing.assert_allclose(c.cpu().numpy(), want_c, rtol=rtol, atol=atol, err_msg=f"dtype {dtype}")
        # masked columns are exactly zero in both h and c
        hz = h.cpu().numpy().reshape(B, H)
        assert np.all(hz[mask == 0] == 0.0) and np.all(c.cpu().numpy().reshape(B, H)[mask == 0] == 0.0)
        # the hidden-to-hidden layer is the same cell on a dense input
        hh = api.Hidden_To_Hidden_Layer(H, dtype=dtype)
        hh.load_weights([t for k, t in enumerate(w) if t is not None and k != 8 and k < 13])
        h2, c2 = hh.forward_prop(dev(h0), dev(mask), dev(h0), dev(c0))
        torch.cuda.synchronize()
        np.testing.assert_allclose(h2.cpu().numpy(), want_h2, rtol=rtol, atol=atol, err_msg=f"dtype {dtype}")
        np.testing.assert_allclose(c2.cpu().numpy(), want_c2, rtol=rtol, atol=atol, err_msg=f"dtype {dtype}")


@pytest.mark.parametrize("att_type,H,B,D,S_max", [(1, 16, 3, 2, 9), (1, 33, 7, 3, 12), (1, 100, 8, 10, 40),
                                                   (1, 256, 64, 10, 80), (2, 16, 3, 0, 9), (2, 33, 7, 0, 12),
                                                   (2, 256, 33, 0, 50)])
def test_attention_matches_oracle(api, oracle, att_type, H, B, D, S_max):
    import torch
    rng = np.random.default_rng(H + B * 17 + att_type)
    sc = 1.0 / np.sqrt(H)
    w6 = [(rng.standard_normal(H * H) * sc).astype(np.float32), (rng.standard_normal(H * H) * sc).astype(np.float32),
          (rng.standard_normal(H) * 0.5).astype(np.float32), (rng.standard_normal(H) * 0.1).astype(np.float32),
          (rng.standard_normal(H * H) * sc).astype(np.float32), (rng.standard_normal(H * H) * sc).astype(np.float32)]
    lens = rng.integers(1, S_max + 1, size=B).astype(np.int32)
    lens[0] = S_max
    if B > 1:
        lens[1] = 1
    offs = (S_max - lens).astype(np.int32)
    hs = (rng.standard_normal(S_max * H * B) * 0.7).astype(np.float32)
    h_t = (rng.standard_normal(H * B) * 0.7).astype(np.float32)
    mask = (rng.random(B) > 0.2).astype(np.int32)
    mask[0] = 1
    want, want_al, want_idx = oracle.attention(att_type, H, B, max(D, 1), w6, h_t, mask, hs, S_max, lens, offs)
    for dtype, rtol, atol in engines_for(H):
        if att_type == 1 and dtype in (1, 2):
            continue  # reduced precision can move floor(p_t) to the next window; covered by the model-level tests
        att = api.attention_layer(H, max(D, 1), att_type, dtype=dtype)
        att.load_weights(w6)
        att.prep_minibatch_info(dev(hs), S_max, B, dev(lens), dev(offs), 1)
        out, al = att.forward_prop(dev(h_t), dev(mask), want_alignments=True)
        torch.cuda.synchronize()
        assert api.lib().zrnn_tc_error() == 0
        np.testing.assert_allclose(al.cpu().numpy(), want_al, rtol=max(rtol, 3e-5), atol=atol, err_msg=f"dtype {dtype}")
        np.testing.assert_allclose(out.cpu().numpy(), want, rtol=max(rtol, 3e-5), atol=max(atol, 3e-6), err_msg=f"dtype {dtype}")
        assert np.all(out.cpu().numpy().reshape(B, H)[mask == 0] == 0.0)
        # viterbi alignment: bit-exact wherever the two largest weights are not within rounding of each other
        _, want_vit = oracle.attention_viterbi(att_type, H, B, max(D, 1), w6, h_t, mask, hs, S_max, lens, offs)
        out2, vit = att.forward_prop_viterbi(dev(h_t), dev(mask))
        torch.cuda.synchronize()
        assert np.array_equal(out2.cpu().numpy(), out.cpu().numpy())
        wal = want_al.reshape(-1, B)
        top2 = np.sort(wal, axis=0)[-2:]
        clear = (top2[1] - top2[0] > 1e-4 * np.abs(top2[1])) | (mask == 0)
        assert np.array_equal(vit.cpu().numpy()[clear], want_vit[clear]), f"dtype {dtype}"
        assert np.all(want_vit[mask == 0] == -1) and clear.mean() > 0.7


def test_attention_shared_source_columns(api, oracle):
    """Decode layout: `beam` consecutive target columns read one source column instead of replicated copies."""
    import torch
    rng = np.random.default_rng(5)
    H, n_sent, beam, S_max, D = 24, 3, 4, 7, 2
    B = n_sent * beam
    for att_type in (1, 2):
        w6 = [(rng.standard_normal(H * H) * 0.2).astype(np.float32) for _ in range(2)] + \
             [(rng.standard_normal(H) * 0.5).astype(np.float32), (rng.standard_normal(H) * 0.1).astype(np.float32)] + \
             [(rng.standard_normal(H * H) * 0.2).astype(np.float32) for _ in range(2)]
        lens = np.array([7, 3, 5], dtype=np.int32)
        offs = (S_max - lens).astype(np.int32)
        hs = (rng.standard_normal(S_max * H * n_sent) * 0.7).astype(np.float32)
        hs_rep = np.repeat(hs.reshape(S_max, n_sent, H), beam, axis=1).reshape(-1)
        h_t = (rng.standard_normal(H * B) * 0.7).astype(np.float32)
        ones = np.ones(B, dtype=np.int32)
        want, _, _ = oracle.attention(att_type, H, B, D, w6, h_t, ones, hs_rep, S_max, np.repeat(lens, beam),
                                      np.repeat(offs, beam))
        att = api.attention_layer(H, D, att_type)
        att.load_weights(w6)
        att.prep_minibatch_info(dev(hs), S_max, n_sent, dev(lens), dev(offs), beam)
        out = att.forward_prop(dev(h_t), None)
        torch.cuda.synchronize()
        np.testing.assert_allclose(out.cpu().numpy(), want, rtol=3e-5, atol=3e-6)


@pytest.mark.parametrize("V,H,N", [(5, 3, 2), (33, 7, 5), (1000, 100, 8), (10000, 100, 280), (5003, 257, 130),
                                   (5003, 256, 300), (20011, 1000, 140)])
def test_softmax_score_matches_oracle(api, oracle, V, H, N):
    import torch
    rng = np.random.default_rng(V + N)
    D = (rng.standard_normal(V * H) / np.sqrt(H)).astype(np.float32)
    b = (rng.standard_normal(V) * 0.1).astype(np.float32)
    h = rng.standard_normal(H * N).astype(np.float32)
    tgt = rng.integers(0, V, size=N).astype(np.int32)
    tgt[0] = V - 1
    mask = (rng.random(N) > 0.2).astype(np.int32)
    want = oracle.softmax_logp(V, H, N, D, b, h, tgt) * mask
    for dtype, rtol, atol in engines_for(H):
        sm = api.softmax_layer(V, H, dtype=dtype)
        sm.load_weights(D, b)
        got = sm.compute_loss(dev(h), dev(tgt), dev(mask))
        torch.cuda.synchronize()
        assert api.lib().zrnn_tc_error() == 0
        if dtype in (3, 4, 5):
            helpers.assert_logp_close(got.cpu().numpy(), want)
        else:
            np.testing.assert_allclose(got.cpu().numpy(), want, rtol=rtol, atol=atol * 3, err_msg=f"dtype {dtype}")
        assert np.all(got.cpu().numpy()[mask == 0] == 0.0)


@pytest.mark.parametrize("dtype", [3, 4, 5])
@pytest.mark.parametrize("G", [2, 3, 8])
def test_vocab_sharded_softmax_equals_unsharded(api, oracle, G, dtype):
    import torch
    rng = np.random.default_rng(G)
    V, H, N = 1003, 64, 37
    D = (rng.standard_normal(V * H) / np.sqrt(H)).astype(np.float32)
    b = (rng.standard_normal(V) * 0.1).astype(np.float32)
    h = rng.standard_normal(H * N).astype(np.float32)
    tgt = rng.integers(0, V, size=N).astype(np.int32)
    mask = np.ones(N, dtype=np.int32)
    want = oracle.softmax_logp(V, H, N, D, b, h, tgt)
    bounds = np.linspace(0, V, G + 1).astype(int)
    parts = []
    for g in range(G):
        sm = api.softmax_layer(V, H, dtype=dtype, shard_lo=int(bounds[g]), shard_hi=int(bounds[g + 1]))
        sm.load_weights(D, b)
        parts.append(sm.partials(dev(h), dev(tgt)))
    mx = torch.stack([p[0] for p in parts])
    sm_ = torch.stack([p[1] for p in parts])
    tg = torch.stack([p[2] for p in parts])
    got = api.softmax_layer.combine(mx, sm_, tg, dev(mask))
    torch.cuda.synchronize()
    helpers.assert_logp_close(got.cpu().numpy(), want)


@pytest.mark.parametrize("V,H,N,k", [(40, 8, 3, 5), (1000, 64, 24, 13), (10007, 100, 70, 13), (50000, 32, 9, 16),
                                     (10007, 1000, 200, 13)])
def test_softmax_topk_matches_oracle(api, oracle, V, H, N, k):
    import torch
    rng = np.random.default_rng(V + k)
    D = (rng.standard_normal(V * H) / np.sqrt(H)).astype(np.float32)
    b = (rng.standard_normal(V) * 0.1).astype(np.float32)
    h = (rng.standard_normal(H * N) * 2).astype(np.float32)
    p = oracle.softmax_dist(V, H, N, D, b, h).reshape(N, V)
    order = np.argsort(-p, axis=1, kind="stable")[:, :k]
    # indices are exact wherever the oracle's neighbouring probabilities are not within float noise of a tie
    sorted_p = np.take_along_axis(p, np.argsort(-p, axis=1, kind="stable")[:, :k + 1], axis=1)
    gaps = (sorted_p[:, :-1] - sorted_p[:, 1:]) / sorted_p[:, :-1]
    for dtype in (3, 4, 5):
        sm = api.softmax_layer(V, H, dtype=dtype)
        sm.load_weights(D, b)
        val, idx, eos = sm.topk(dev(h), k)
        torch.cuda.synchronize()
        assert api.lib().zrnn_tc_error() == 0
        val, idx, eos = val.cpu().numpy(), idx.cpu().numpy(), eos.cpu().numpy()
        clear = gaps.min(axis=1) > (1e-5 if dtype == 3 else 2e-4)
        assert clear.sum() >= N // 2
        assert np.array_equal(idx[clear], order[clear])
        want = np.log(np.take_along_axis(p, idx.astype(np.int64), axis=1).astype(np.float64))
        np.testing.assert_allclose(val, want, rtol=2e-5, atol=5e-5)
        np.testing.assert_allclose(eos, np.log(p[:, 1].astype(np.float64)), rtol=2e-5, atol=5e-5)
        assert np.all(np.diff(val, axis=1) <= 0)
