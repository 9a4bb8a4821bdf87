"""ScalarQuantizer / BinaryQuantizer kernels against the CPU oracle, bit for bit."""
import numpy as np
import pytest

import vq_b200 as vq
from vq_b200 import synth

pytestmark = pytest.mark.gpu

SPECIALS = np.array([np.nan, np.inf, -np.inf, 0.0, -0.0, 1.0, -1.0, 0.5, 1e-45, -1e-45, 3.4e38, -3.4e38, 0.49999997, 0.50000006],
                    np.float32)


@pytest.mark.parametrize("n", [0, 1, 15, 16, 17, 1000, 4097, 1 << 20])
def test_sq_bq_sizes(oracle, n):
    x = synth.uniform(max(n, 1), 1, 3, -1.5, 1.5).reshape(-1)[:n]
    if n >= len(SPECIALS):
        x[: len(SPECIALS)] = SPECIALS
    for (lo, hi, levels) in ((0.0, 1.0, 256), (-1.0, 1.0, 5), (-0.25, 0.75, 2), (-1000.0, 1000.0, 256)):
        q = vq.ScalarQuantizer.fit(lo, hi, levels)
        assert q.step == oracle.sq_fit(lo, hi, levels)
        assert np.array_equal(q.quantize(x), oracle.sq_quantize(lo, hi, levels, q.step, x))
    for (thr, low, high) in ((0.0, 0, 1), (0.5, 3, 200), (-0.1, 0, 255)):
        b = vq.BinaryQuantizer.fit(thr, low, high)
        assert np.array_equal(b.quantize(x), oracle.bq_quantize(thr, low, high, x))


def test_vector_shapes_like_the_reference_api(oracle):
    x = synth.uniform(100, 1024, 42, -1000.0, 1000.0)  # tests/test_sq.rs:36-77 shape
    q = vq.ScalarQuantizer.fit(-1000.0, 1000.0, 256)
    for row in x[:5]:
        idx = q.quantize(row)
        assert idx.shape == (1024,) and idx.dtype == np.uint8
        assert np.array_equal(idx, oracle.sq_quantize(-1000.0, 1000.0, 256, q.step, row))
    assert q.quantize(x).shape == x.shape


def test_unaligned_device_pointers(oracle):
    import torch
    x = synth.uniform(1, 100003, 9, -1.0, 2.0).reshape(-1)
    buf = torch.empty(x.size + 8, device="cuda")
    q = vq.ScalarQuantizer.fit(0.0, 1.0, 256)
    b = vq.BinaryQuantizer.fit(0.25, 1, 2)
    for off in (0, 1, 3, 4):
        view = buf[off:off + x.size]
        view.copy_(torch.from_numpy(x))
        assert np.array_equal(q.quantize(view).cpu().numpy(), oracle.sq_quantize(0.0, 1.0, 256, q.step, x))
        assert np.array_equal(b.quantize(view).cpu().numpy(), oracle.bq_quantize(0.25, 1, 2, x))


def test_full_size_10m_x_128(oracle):
    """The element-wise benchmark configuration: 10,000,000 x 128 values in [-1, 1); SQ [0,1] with 256 levels, BQ threshold 0.
    Device-generated (seeded torch generator) to avoid a 5 GB host array; whole-array properties plus oracle
    comparison on sampled slabs."""
    import torch
    n = 10_000_000 * 128
    g = torch.Generator(device="cuda")
    g.manual_seed(1)
    x = torch.empty(n, device="cuda", dtype=torch.float32)
    x.uniform_(-1.0, 1.0, generator=g)
    q = vq.ScalarQuantizer.fit(0.0, 1.0, 256)
    b = vq.BinaryQuantizer.fit(0.0, 0, 1)
    sq = q.quantize(x)
    bq = b.quantize(x)
    assert sq.shape == x.shape and bq.shape == x.shape
    # BQ is exactly the comparison, everywhere
    assert torch.equal(bq, (x >= 0).to(torch.uint8))
    # SQ: negative inputs clamp to level 0; monotone in x; reconstruction within half a step (+2 ulp)
    assert int(sq[x < 0].max()) == 0
    recon = sq.float() * q.step
    err = (recon - x.clamp(0.0, 1.0)).abs().max().item()
    assert err <= q.step / 2 + 2.4e-7
    # checksum of checksums: histogram must match the oracle's on sampled slabs, and slabs bit for bit
    rng = np.random.default_rng(0)
    for start in rng.integers(0, n - (1 << 20), 12):
        sl = x[start:start + (1 << 20)].cpu().numpy()
        assert np.array_equal(sq[start:start + (1 << 20)].cpu().numpy(), oracle.sq_quantize(0.0, 1.0, 256, q.step, sl))
        assert np.array_equal(bq[start:start + (1 << 20)].cpu().numpy(), oracle.bq_quantize(0.0, 0, 1, sl))


def test_large_host_arrays_go_through_the_chunked_pipeline(oracle):
    n = (1 << 24) + 12345  # just over two 8 Mi-value chunks
    x = synth.uniform(n, 1, 5, -1.5, 1.5).reshape(-1)
    q = vq.ScalarQuantizer.fit(0.0, 1.0, 256)
    assert np.array_equal(q.quantize(x), oracle.sq_quantize(0.0, 1.0, 256, q.step, x))
    b = vq.BinaryQuantizer.fit(0.1, 2, 7)
    assert np.array_equal(b.quantize(x), oracle.bq_quantize(0.1, 2, 7, x))
