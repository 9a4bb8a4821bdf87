"""Tree-structured VQ (src/tsvq.rs): the oracle against an independent transcription and the reference's own test
(tests/test_tsvq.rs:11-22); the device build and lookup against the oracle, bit for bit."""
import numpy as np
import pytest

import oracle
from tests.golden import reference_known_answers as ka
from vq_b200 import synth


def _recursive_fit(x, max_depth):
    """Plain-Python transcription of TSVQNode::fit (src/tsvq.rs:71-148), recursive like the reference."""
    x = np.asarray(x, np.float32)
    dim = x.shape[1]
    c = np.zeros(dim, np.float32)
    for i0 in range(0, len(x), 1024):        # sums of consecutive 1024-row chunks; one chunk = the reference's serial sum
        part = np.zeros(dim, np.float32)
        for row in x[i0:i0 + 1024]:
            part = part + row
        c = c + part
    c = c / np.float32(len(x))
    node = {"c": c, "l": None, "r": None}
    if max_depth == 0 or len(x) <= 1:
        return node
    var = np.zeros(dim, np.float32)
    for row in x:
        d = row - c
        var = var + d * d
    split = 0
    for t in range(1, dim):
        if not (var[t] < var[split]):        # max_by keeps the last of equal maxima
            split = t
    vals = np.sort(x[:, split], kind="stable")
    n = len(vals)
    med = np.float32((vals[n // 2 - 1] + vals[n // 2]) / np.float32(2.0)) if n % 2 == 0 else vals[n // 2]
    mask = x[:, split] <= med
    lo, hi = x[mask], x[~mask]
    if 0 < len(lo) < n:
        node["l"] = _recursive_fit(lo, max_depth - 1)
    if 0 < len(hi) < n:
        node["r"] = _recursive_fit(hi, max_depth - 1)
    return node


def _bfs(root):
    order, cents, left, right = [root], [], [], []
    i = 0
    while i < len(order):
        nd = order[i]
        cents.append(nd["c"])
        for side, dst in (("l", left), ("r", right)):
            if nd[side] is not None:
                dst.append(len(order))
                order.append(nd[side])
            else:
                dst.append(-1)
        i += 1
    return np.stack(cents), np.array(left, np.int32), np.array(right, np.int32)


@pytest.mark.parametrize("n,dim,depth,seed", [(1, 3, 5, 0), (2, 4, 0, 1), (50, 6, 3, 2), (333, 10, 6, 3), (1000, 10, 3, 4), (257, 5, 12, 5),
                                              (2500, 4, 2, 6)])
def test_oracle_tree_equals_the_recursive_transcription(n, dim, depth, seed):
    x = synth.normal(n, dim, seed)
    x[::7] = x[0]                                    # duplicates: equal values around the median
    c, l, r = oracle.tsvq_fit(x, depth)
    c2, l2, r2 = _bfs(_recursive_fit(x, depth))
    assert np.array_equal(l, l2) and np.array_equal(r, r2)
    assert np.array_equal(c, c2)


def test_oracle_identical_vectors_round_trip():
    """tests/test_tsvq.rs:11-22: ten copies of one vector, depth 3: the quantized vector equals it within 1e-6."""
    v = np.array([1.0, 2.0, 3.0, 4.0, 5.0], np.float32)
    x = np.tile(v, (10, 1))
    c, l, r = oracle.tsvq_fit(x, 3)
    assert len(c) == 1 and l[0] == -1 and r[0] == -1   # nothing can be split
    out, leaf = oracle.tsvq_quantize(c, l, r, v[None], ka.SQ)
    assert np.abs(out.view(np.float16).astype(np.float32)[0] - v).max() < 1e-6


def test_oracle_rejects_empty_and_nan():
    with pytest.raises(oracle.OracleError, match="Empty input"):
        oracle.tsvq_fit(np.zeros((0, 4), np.float32), 3)
    x = synth.normal(20, 3, 1)
    x[4, 1] = np.nan
    with pytest.raises(oracle.OracleError):
        oracle.tsvq_fit(x, 3)


# ---------------------------------------------------------------------------------------------- device
@pytest.mark.gpu
@pytest.mark.parametrize("n,dim,depth,seed", [(1, 3, 5, 0), (2, 4, 0, 1), (50, 6, 3, 2), (333, 10, 6, 3), (1000, 10, 3, 4), (257, 5, 12, 5),
                                              (5000, 128, 10, 6), (70000, 33, 8, 7),
                                              # widths in whole 128-byte pieces take the streaming statistics kernel: stage edges, tails
                                              (64, 32, 2, 8), (65, 32, 3, 9), (1537, 96, 4, 10), (100000, 64, 9, 11), (200001, 128, 6, 12)])
def test_device_tree_and_lookup_equal_the_oracle(n, dim, depth, seed):
    import vq_b200 as vq

    x = synth.normal(n, dim, seed)
    x[::7] = x[0]
    c, l, r = oracle.tsvq_fit(x, depth)
    t = vq.TSVQ(x, depth, vq.Distance.Euclidean)
    cg, lg, rg = t.tree()
    assert np.array_equal(lg, l) and np.array_equal(rg, r)
    assert np.array_equal(cg, c)
    q = synth.normal(2000, dim, seed + 100)
    out, leaf = t.quantize(q, return_leaf=True)
    out_o, leaf_o = oracle.tsvq_quantize(c, l, r, q, ka.EUCLID)
    assert np.array_equal(leaf, leaf_o)
    assert np.array_equal(np.asarray(out).view(np.uint16), out_o)


@pytest.mark.gpu
@pytest.mark.parametrize("metric", ["SquaredEuclidean", "CosineDistance", "Manhattan", "Chebyshev", "Hamming"])
def test_device_lookup_all_metrics(metric):
    import vq_b200 as vq

    x = synth.normal(3000, 16, 11)
    d = getattr(vq.Distance, metric)
    t = vq.TSVQ(x, 7, d)
    c, l, r = t.tree()
    q = synth.normal(1500, 16, 12)
    q[5] = 0.0                                        # zero norm: cosine distance 1 to both children -> left
    _, leaf = t.quantize(q, return_leaf=True)
    _, leaf_o = oracle.tsvq_quantize(c, l, r, q, d.metric, d.p)
    assert np.array_equal(leaf, leaf_o)


@pytest.mark.gpu
def test_device_reference_cases_and_errors():
    import torch

    import vq_b200 as vq

    v = np.array([1.0, 2.0, 3.0, 4.0, 5.0], np.float32)
    t = vq.TSVQ(np.tile(v, (10, 1)), 3, vq.Distance.SquaredEuclidean)          # tests/test_tsvq.rs:11-22
    assert np.abs(np.asarray(t.quantize(v)).astype(np.float32) - v).max() < 1e-6
    with pytest.raises(vq.EmptyInput):
        vq.TSVQ(np.zeros((0, 5), np.float32), 3, vq.Distance.Euclidean)
    with pytest.raises(vq.DimensionMismatch, match="expected 5, got 4"):
        t.quantize(np.zeros(4, np.float32))
    bad = synth.normal(100, 4, 3)
    bad[17, 2] = np.nan
    with pytest.raises(vq.VqError):
        vq.TSVQ(bad, 4, vq.Distance.Euclidean)
    # device-resident input and output
    x = torch.from_numpy(synth.normal(4096, 32, 5)).cuda()
    t2 = vq.TSVQ(x, 6, vq.Distance.Euclidean)
    out = t2.quantize(x)
    assert out.is_cuda and out.shape == (4096, 32)
    c, l, r = t2.tree()
    out_o, _ = oracle.tsvq_quantize(c, l, r, x.cpu().numpy(), ka.EUCLID)
    assert np.array_equal(out.cpu().numpy().view(np.uint16), out_o)
