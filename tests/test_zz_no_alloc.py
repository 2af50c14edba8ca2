"""The allocation-free scoring softmax (zrnn_softmax_score_noalloc) against the regular entry point.

Some callers cannot allocate device memory while they run (their own arena owns the GPU, or they cannot take
the device-wide stall of cudaMalloc), so this entry point works out of a fixed array inside the library.  The
file name sorts last on purpose: with `pytest -x` every other test has already run if this one fails.
"""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [0, 1])  # an fp32 layer and a bf16 layer
def test_noalloc_softmax_matches_regular_entry_point_twice(oracle, dtype):
    import torch
    assert torch.cuda.is_available(), "needs a CUDA device"
    from tests import helpers
    from zoph_rnn_b200 import api
    rng = np.random.default_rng(123)
    V, H = 5003, 96
    D = (rng.standard_normal(V * H) / np.sqrt(H)).astype(np.float32)
    b = (rng.standard_normal(V) * 0.1).astype(np.float32)
    sm = api.softmax_layer(V, H, dtype=dtype)
    sm.load_weights(D, b)
    # two calls in a row with different sizes and data: the second one finds the first one's numbers in the
    # shared scratch array and must not be affected by them
    for call, N in enumerate((130, 37)):
        h = torch.as_tensor(rng.standard_normal(H * N).astype(np.float32)).cuda()
        tgt = torch.as_tensor(rng.integers(0, V, size=N).astype(np.int32)).cuda()
        mask = torch.as_tensor((rng.random(N) > 0.2).astype(np.int32)).cuda()
        want = sm.compute_loss(h, tgt, mask)
        out = torch.full((N,), 7.0, dtype=torch.float32, device="cuda")
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        got = sm.compute_loss_noalloc(h, tgt, mask, out)
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        # the first call on a device is the set-up call: it looks the array up and the driver may place the
        # library's image (the 16 MiB array included) on the GPU at that moment; later calls must take nothing
        if call > 0:
            assert free_after >= free_before, "the allocation-free entry point took device memory"
        # the entry point always computes in fp32 FMA on the layer's fp32 weights, whatever the layer's dtype: it
        # matches the CPU oracle at the fp32 tolerance, and the regular entry point at that layer's own tolerance
        mk = mask.cpu().numpy()
        ref = oracle.softmax_logp(V, H, N, D, b, h.cpu().numpy(), tgt.cpu().numpy()) * mk
        helpers.assert_logp_close(got.cpu().numpy(), ref)
        if dtype == 0:
            helpers.assert_logp_close(got.cpu().numpy(), want.cpu().numpy())
        else:
            assert np.abs(got.cpu().numpy() - want.cpu().numpy()).max() < 0.05
        assert np.all(got.cpu().numpy()[mk == 0] == 0.0)


def test_noalloc_softmax_rejects_oversized_requests():
    import torch
    assert torch.cuda.is_available(), "needs a CUDA device"
    from zoph_rnn_b200 import api
    V, H = 20000, 8
    sm = api.softmax_layer(V, H)
    sm.load_weights(np.zeros(V * H, np.float32), np.zeros(V, np.float32))
    limit = api.lib().zrnn_softmax_score_noalloc_max_floats()
    N = limit // (2 * ((V + 127) // 128) + 1) + 1  # one column too many
    h = torch.zeros(H * N, dtype=torch.float32, device="cuda")
    tgt = torch.zeros(N, dtype=torch.int32, device="cuda")
    out = torch.empty(N, dtype=torch.float32, device="cuda")
    with pytest.raises(api.ZrnnError) as e:
        sm.compute_loss_noalloc(h, tgt, None, out)
    assert e.value.status == 1 and "scratch floats" in str(e.value)
    sm.compute_loss_noalloc(h[: H * (N - 1)], tgt[: N - 1], None, out[: N - 1])  # exactly at the limit: accepted
    torch.cuda.synchronize()
