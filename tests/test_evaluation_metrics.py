"""The evaluation metrics of the reference's harness (src/bin/utils.rs:50-127): oracle on CPU, device parity on GPU."""
import numpy as np
import pytest

import oracle
from vq_b200 import synth


def _noisy_f16(x, scale, seed):
    rng = np.random.default_rng(seed)
    return (x + rng.normal(0, scale, x.shape).astype(np.float32)).astype(np.float16)


def test_oracle_recall_identity_and_noise():
    x = synth.uniform01(600, 16, seed=3)
    assert oracle.recall_at_k(x, x.copy(), 10) == pytest.approx(1.0)
    q = _noisy_f16(x, 0.5, 1).astype(np.float32)
    r = oracle.recall_at_k(x, q, 10)
    assert 0.0 <= r < 0.9


def test_oracle_recall_window_excludes_far_rows():
    # 12000 rows > 10000: each query only sees 5000 rows around it; duplicates of the query outside the window never count
    n, d = 12000, 4
    x = synth.uniform01(n, d, seed=5)
    x[11000] = x[0]  # outside row 0's window [0, 2500)
    approx = x.copy()
    assert oracle.recall_at_k(x, approx, 10) == pytest.approx(1.0)
    # divisor is n // step while ceil(n / step) queries are summed (src/bin/utils.rs:79,126)
    n2 = 1500
    x2 = synth.uniform01(n2, d, seed=6)
    assert oracle.recall_at_k(x2, x2.copy(), 5) == pytest.approx(1.0)


@pytest.mark.gpu
@pytest.mark.parametrize("n,dim,k", [(700, 16, 10), (1500, 32, 10), (12000, 24, 10), (2500, 128, 5), (64, 8, 32)])
def test_device_metrics_match_oracle(n, dim, k):
    import vq_b200 as vq

    x = synth.uniform01(n, dim, seed=n)
    q = _noisy_f16(x, 0.08, n + 1)
    mse, rec = vq.evaluate(x, q, k)
    want_mse = oracle.mse_f16(x, q.view(np.uint16))
    want_rec = oracle.recall_at_k(x, q.astype(np.float32), k)
    assert mse == pytest.approx(want_mse, rel=1e-5)
    assert rec == want_rec  # integer hit counts summed in the same f32 order


@pytest.mark.gpu
def test_device_metrics_with_ties_and_device_tensors():
    import torch

    import vq_b200 as vq

    # a coarse reconstruction: many rows share one reconstructed vector, so approximate distances tie and the
    # lowest row index must win, as the reference's stable sort does
    n, dim = 3000, 16
    x = synth.uniform01(n, dim, seed=9)
    q = (np.round(x * 2) / 2).astype(np.float16)
    xd = torch.from_numpy(x).cuda()
    qd = torch.from_numpy(q).cuda()
    mse, rec = vq.evaluate(xd, qd, 10)
    assert rec == oracle.recall_at_k(x, q.astype(np.float32), 10)
    assert mse == pytest.approx(oracle.mse_f16(x, q.view(np.uint16)), rel=1e-5)


@pytest.mark.gpu
def test_device_metrics_on_pq_output():
    import vq_b200 as vq

    x = synth.gaussian_mixture(20000, 32, seed=4, components=16)
    pq = vq.ProductQuantizer.fit(x[:5000], 4, 16, 5, vq.Distance.SquaredEuclidean, 42)
    q = pq.quantize(x)
    mse, rec = vq.evaluate(x, q, 10)
    assert mse == pytest.approx(oracle.mse_f16(x, np.asarray(q).view(np.uint16)), rel=1e-5)
    assert rec == oracle.recall_at_k(x, np.asarray(q).astype(np.float32), 10)


@pytest.mark.gpu
def test_device_metrics_reject_bad_k():
    import vq_b200 as vq

    x = synth.uniform01(100, 8, seed=1)
    with pytest.raises(vq.VqError):
        vq.evaluate(x, x.astype(np.float16), 0)
    with pytest.raises(vq.VqError):
        vq.evaluate(x, x.astype(np.float16), 33)
