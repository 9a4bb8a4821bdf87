"""The two dense contractions of OPQ on the tensor cores (split-TF32 tcgen05 kernels) against f64.

y = R x (src/opq.rs:186-194, 232-234) and A = sum_r y_r x_r^T (src/opq.rs:172-179).  The reference computes both in f32
with nalgebra, whose summation order is not pinned, so the bar is f32-level accuracy, stated here against an f64 product:
every entry within 4e-6 * sum_i |a_i b_i| (about sixteen times the error an f32 chain of this length makes), which is what
keeps the rotated rows -- and with them the codes -- at rounding distance from any f32 implementation.
"""
import ctypes as C

import numpy as np
import pytest

import vq_b200 as vq
from vq_b200 import _lib

pytestmark = pytest.mark.gpu


def _rotate(ctx, rot, x):
    y = np.empty_like(x)
    rc = _lib.load().vqb_opq_rotate_rows(ctx.handle, rot.ctypes.data, rot.shape[0], x.ctypes.data, x.shape[0], y.ctypes.data)
    assert rc == 0, _lib.load().vqb_last_error(ctx.handle)
    return y


def _cross(ctx, y, x):
    a = np.empty((x.shape[1], x.shape[1]), np.float64)
    rc = _lib.load().vqb_opq_cross_cov(ctx.handle, y.ctypes.data, x.ctypes.data, x.shape[0], x.shape[1], a.ctypes.data)
    assert rc == 0, _lib.load().vqb_last_error(ctx.handle)
    return a


@pytest.mark.parametrize("dim,n", [(128, 1000), (128, 128 * 148 * 2 + 77), (64, 5000), (32, 333), (96, 4097)])
def test_rotation_has_f32_accuracy(ctx, dim, n):
    rng = np.random.default_rng(dim + n)
    q, _ = np.linalg.qr(rng.normal(size=(dim, dim)))
    rot = np.ascontiguousarray(q.astype(np.float32))
    x = (rng.normal(size=(n, dim)) * rng.uniform(0.01, 30.0, size=(n, 1))).astype(np.float32)
    y = _rotate(ctx, rot, x)
    exact = x.astype(np.float64) @ rot.astype(np.float64).T
    scale = np.abs(x).astype(np.float64) @ np.abs(rot).astype(np.float64).T
    assert np.abs(y - exact).max() <= 4e-6 * scale.max()
    assert (np.abs(y - exact) <= 4e-6 * scale + 1e-30).all()


def test_rotation_of_exactly_representable_values_is_exact(ctx):
    """Small integers and a permutation-with-signs matrix: every product and every sum is exact, so the result must be too."""
    rng = np.random.default_rng(3)
    dim, n = 128, 3000
    perm = rng.permutation(dim)
    rot = np.zeros((dim, dim), np.float32)
    rot[np.arange(dim), perm] = rng.choice([-1.0, 1.0], dim)
    x = rng.integers(-2000, 2000, (n, dim)).astype(np.float32) + rng.integers(0, 4096, (n, dim)).astype(np.float32) / 4096.0
    y = _rotate(ctx, rot, x)
    assert np.array_equal(y, x[:, perm] * rot[np.arange(dim), perm])


@pytest.mark.parametrize("dim,n", [(128, 4096 * 3 + 5), (128, 200_003), (64, 10_000), (32, 31), (96, 5000)])
def test_cross_covariance_has_f32_accuracy(ctx, dim, n):
    rng = np.random.default_rng(7 * dim + n)
    x = rng.normal(size=(n, dim)).astype(np.float32)
    y = (x + 0.1 * rng.normal(size=(n, dim))).astype(np.float32)
    a = _cross(ctx, y, x)
    exact = y.astype(np.float64).T @ x.astype(np.float64)
    scale = np.abs(y).astype(np.float64).T @ np.abs(x).astype(np.float64)
    assert (np.abs(a - exact) <= 4e-6 * scale + 1e-30).all(), float((np.abs(a - exact) / scale).max())


def test_other_widths_take_the_fp32_kernels(ctx):
    rng = np.random.default_rng(1)
    dim, n = 20, 700
    q, _ = np.linalg.qr(rng.normal(size=(dim, dim)))
    rot = np.ascontiguousarray(q.astype(np.float32))
    x = rng.normal(size=(n, dim)).astype(np.float32)
    y = _rotate(ctx, rot, x)
    assert np.allclose(y, x @ rot.T, atol=1e-5)
    a = _cross(ctx, y, x)
    assert np.allclose(a, y.astype(np.float64).T @ x.astype(np.float64), rtol=1e-5, atol=1e-3)
