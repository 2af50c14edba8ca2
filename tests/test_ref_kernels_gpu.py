"""Pins the CPU oracle to the reference's own code: the reference's kernel file (src/custom_kernels.h), compiled
unmodified for sm_100a behind oracle/ref_shim.cu and launched with the reference's own grid / block shapes
(src/LSTM.hpp:89-399, src/attention_node.hpp:141-379, src/Input_To_Hidden_Layer.hpp:1196-1202,
src/softmax.hpp:658-661), against the oracle's restatement of the same steps.

The matrix products between those kernels are cuBLAS calls in the reference (plain fp32 products); a naive
double-accumulating kernel stands in for them on the reference side, as the oracle does on its side, so the compared
quantities differ only by what the element-wise and attention kernels compute.  Not covered: the two softmax
distribution kernels, whose `volatile` warp reductions are only defined for lock-step warps (src/custom_kernels.h:
454-474); the oracle's log-softmax is checked against the float64 NumPy witness instead (tests/test_oracle_cpu.py).
"""
import numpy as np
import pytest

from oracle import ref_kernels

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref():
    import torch
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    assert ref_kernels.available(), ("oracle/_ref/libzoph_ref_kernels.so is missing: build it where the reference's "
                                     "sources are present (make -C oracle ref)")
    return ref_kernels


def rand_lstm17(rng, H, feed, scale):
    w = [None] * 17
    for g in range(4):
        w[2 * g] = (rng.standard_normal(H * H) * scale).astype(np.float32)
        w[2 * g + 1] = (rng.standard_normal(H) * 0.3).astype(np.float32)
    for k in range(9, 17 if feed else 13):
        w[k] = (rng.standard_normal(H * H) * scale).astype(np.float32)
    return w


def test_id_preparation(ref):
    """vocab_to_01 / vocab_to_nonM1 (src/custom_kernels.h:9-32) against the rule the oracle and the product apply."""
    rng = np.random.default_rng(1)
    ids = rng.integers(-1, 50, size=20011).astype(np.int32)
    nonm1, m01 = ref.prep_vocab(ids)
    assert np.array_equal(nonm1, np.where(ids == -1, 0, ids))
    assert np.array_equal(m01, (ids != -1).astype(np.int32))


@pytest.mark.parametrize("H,V,n", [(1, 5, 3), (100, 1000, 64), (1000, 3000, 128)])
def test_embedding_lookup(ref, oracle, H, V, n):
    """sparse_lookup_kernel (src/custom_kernels.h:340-348) against the oracle's gather, bit for bit."""
    rng = np.random.default_rng(H + V)
    W = rng.standard_normal(H * V).astype(np.float32)
    ids = rng.integers(0, V, size=n).astype(np.int32)
    got = ref.sparse_lookup(W, H, V, ids)
    want = oracle.gather(W, H, ids)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_bias_add(ref):
    """matrix_bias_kernel (src/custom_kernels.h:785-794): z[v, n] += b_d[v], the step between the vocabulary GEMM
    and the log-softmax that the oracle performs as `zc[v] + b_d[v]`."""
    rng = np.random.default_rng(3)
    V, N = 1003, 7
    z = rng.standard_normal(V * N).astype(np.float32)
    b = rng.standard_normal(V).astype(np.float32)
    got = ref.matrix_bias(V, N, z, b)
    assert np.array_equal(got, (z.reshape(N, V) + b[None, :]).reshape(-1))


@pytest.mark.parametrize("H,B,feed", [(3, 2, False), (33, 5, True), (100, 8, False), (256, 70, True), (1000, 16, True),
                                       (1000, 128, False)])
def test_lstm_cell(ref, oracle, H, B, feed):
    """forward_sigmoid_kernel(_feed), forward_tanh_kernel(_feed), forward_c_t_kernel, forward_h_t_kernel and
    zero_c_t_and_h_t in the order of LSTM_IH_Node::forward_prop_GPU against the oracle's lstm_cell."""
    rng = np.random.default_rng(H * 17 + B)
    w = rand_lstm17(rng, H, feed, 0.6 / np.sqrt(H))
    x, h0, c0 = (rng.standard_normal(H * B).astype(np.float32) * 0.6 for _ in range(3))
    ht = rng.standard_normal(H * B).astype(np.float32) * 0.6 if feed else None
    mask = (rng.random(B) > 0.25).astype(np.int32)
    mask[0] = 1
    got_h, got_c = ref.lstm_cell(H, B, w, x, h0, c0, ht, mask)
    want_h, want_c = oracle.lstm_cell(H, B, w, x, h0, c0, ht, mask)
    # both sides form the pre-activations from double-accumulated products rounded to fp32; what is left is one
    # fp32 rounding in the order of the three-term sums and libm vs. device math functions (a few ulp)
    np.testing.assert_allclose(got_h, want_h, rtol=5e-6, atol=1e-6)
    np.testing.assert_allclose(got_c, want_c, rtol=5e-6, atol=1e-6)
    hz = got_h.reshape(B, H)
    assert np.all(hz[mask == 0] == 0.0) and np.all(got_c.reshape(B, H)[mask == 0] == 0.0)


@pytest.mark.parametrize("H,B,D,S_max", [(8, 3, 2, 7), (100, 9, 3, 25), (256, 33, 10, 80), (1000, 16, 10, 50)])
def test_local_p_attention(ref, oracle, H, B, D, S_max):
    """tanh_kernel, sigmoid_kernel, alignment_pos_kernel, lower_upper_kernel, create_indicies_kernel, load_in_hs_kernel,
    elem_reduce_kernel_large, alignment_reduction_kernel, get_viterbi_alignment_kernel, create_c_t_kernel,
    tanh_att_forward_kernel and zero_h_t in the order of attention_node::forward_prop against the oracle's attention
    step: window indices and viterbi alignments exactly, weights and output within fp32 rounding."""
    rng = np.random.default_rng(H + 7 * B + D)
    sc = 1.0 / np.sqrt(H)
    w6 = [(rng.standard_normal(H * H) * 0.3 * sc).astype(np.float32), (rng.standard_normal(H * H) * sc).astype(np.float32),
          (rng.standard_normal(H) * 2.0 * sc).astype(np.float32), (rng.standard_normal(H) * 0.3).astype(np.float32),
          (rng.standard_normal(H * H) * sc).astype(np.float32), (rng.standard_normal(H * H) * sc).astype(np.float32)]
    h_t = rng.standard_normal(H * B).astype(np.float32)
    lens = rng.integers(1, S_max + 1, size=B).astype(np.int32)
    lens[0] = S_max
    offs = (S_max - lens).astype(np.int32)
    mask = (rng.random(B) > 0.2).astype(np.int32)
    mask[0] = 1
    hs = (rng.standard_normal(S_max * H * B) * 0.7).astype(np.float32).reshape(S_max, B, H)
    for b in range(B):  # left-padded source columns are exactly zero until the sentence starts
        hs[:offs[b], b, :] = 0.0
    got_out, got_al, got_idx, got_p, got_vit = ref.attention_localp(H, B, D, w6, h_t, mask, hs, S_max, lens, offs)
    want_out, want_al, want_idx = oracle.attention(1, H, B, D, w6, h_t, mask, hs, S_max, lens, offs)
    _, want_vit = oracle.attention_viterbi(1, H, B, D, w6, h_t, mask, hs, S_max, lens, offs)
    # a p_t within rounding of an integer could truncate differently on the two sides; such inputs are regenerated
    # by the seed choice, not tolerated
    frac = got_p - np.floor(got_p)
    assert np.all((frac > 1e-4) & (frac < 1 - 1e-4) | (mask == 0)), "test input has p_t next to an integer"
    assert np.array_equal(got_idx, want_idx)
    # scores: fp32 tree reduction (reference) against a double sum (oracle), then exp of scores of magnitude ~5
    np.testing.assert_allclose(got_al, want_al, rtol=5e-5, atol=1e-7)
    np.testing.assert_allclose(got_out, want_out, rtol=2e-5, atol=5e-6)
    live = mask == 1
    assert np.array_equal(got_vit[live], want_vit[live])
    assert np.all(got_out.reshape(B, H)[~live] == 0.0)
