"""The tcgen05 tensor-core GEMM building block against a float64 product, through the C ABI."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

# relative tolerances on |C - C_ref| / (|W| |X|) row-column norms (summation-independent scale)
TOL = {0: 2e-6, 1: 8e-3, 2: 1.5e-3, 3: 4e-6, 4: 4e-6}


@pytest.mark.parametrize("mode", [0, 1, 2, 3, 4])
@pytest.mark.parametrize("n,m,k", [(32, 128, 64), (128, 128, 256), (100, 7, 100), (1000, 128, 1000), (4000, 200, 2000),
                                   (333, 130, 77)])
def test_gemm_modes(mode, n, m, k):
    import torch
    assert torch.cuda.is_available()
    from zoph_rnn_b200 import api
    rng = np.random.default_rng(n + m + k)
    W = rng.standard_normal((k, n)).astype(np.float32) * 0.1   # column-major n x k stored as [k][n]
    X = rng.standard_normal((m, k)).astype(np.float32)          # column-major k x m stored as [m][k]
    C = api.gemm(torch.as_tensor(W).cuda().reshape(-1), torch.as_tensor(X).cuda().reshape(-1), n, m, k, mode)
    torch.cuda.synchronize()
    got = C.cpu().numpy().reshape(m, n)
    want = X.astype(np.float64) @ W.astype(np.float64)
    scale = np.linalg.norm(X.astype(np.float64), axis=1)[:, None] * np.linalg.norm(W.astype(np.float64), axis=0)[None, :]
    err = np.abs(got - want) / scale
    assert err.max() < TOL[mode], f"mode {mode}: max scaled error {err.max():.3e}"
