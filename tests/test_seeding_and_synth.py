"""Host logic: the stand-in sampler, shard arithmetic and the synthetic generators."""
import numpy as np

from vq_b200 import synth
from vq_b200.distributed import owner_of, shard_bounds
from vq_b200.seeding import LbgSeeder, StandInRng


def test_splitmix_reference_values():
    # SplitMix64 with seed 0: first outputs of the published algorithm
    r = StandInRng(0)
    assert [r.next_u64() for _ in range(3)] == [0xE220A8397B1DCDAF, 0x6E789E6AA1B965F4, 0x06C45D188009454F]


def test_choose_multiple_is_a_sample_without_replacement():
    r = StandInRng(42)
    idx = r.choose_multiple(1000, 256)
    assert len(set(idx.tolist())) == 256 and idx.max() < 1000
    assert np.array_equal(idx, StandInRng(42).choose_multiple(1000, 256))
    assert sorted(StandInRng(1).choose_multiple(5, 5).tolist()) == [0, 1, 2, 3, 4]


def test_seeder_streams_follow_seed_plus_index():
    s = LbgSeeder(100)
    a = s.init_indices(3, 500, 8)
    assert np.array_equal(a, StandInRng(103).choose_multiple(500, 8))
    ref = StandInRng(103)
    ref.choose_multiple(500, 8)
    assert s.draw(3, 500) == ref.choose(500)


def test_shard_bounds_cover_and_owner():
    for n in (0, 1, 7, 10, 1000003):
        for w in (1, 2, 3, 8):
            edges = [shard_bounds(n, r, w) for r in range(w)]
            assert edges[0][0] == 0 and edges[-1][1] == n
            assert all(edges[r][1] == edges[r + 1][0] for r in range(w - 1))
            for row in {0, n // 2, max(n - 1, 0)} if n else set():
                r = owner_of(row, n, w)
                assert edges[r][0] <= row < edges[r][1]


def test_uniform_generator_is_deterministic_and_in_range():
    a = synth.uniform01(1000, 16, 7)
    assert a.dtype == np.float32 and a.shape == (1000, 16)
    assert a.min() >= 0.0 and a.max() < 1.0
    assert np.array_equal(a, synth.uniform01(1000, 16, 7, chunk_rows=13))
    assert abs(float(a.mean()) - 0.5) < 0.02
    b = synth.uniform(100, 8, 1, -1.0, 1.0)
    assert b.min() >= -1.0 and b.max() < 1.0


def test_other_generators_shapes():
    g = synth.gaussian_mixture(2000, 16, 11)
    assert g.shape == (2000, 16) and np.isfinite(g).all()
    c = synth.correlated(500, 8, 3)
    assert c.shape == (500, 8) and np.isfinite(c).all()
    z = synth.normal(20000, 4, 9)
    assert abs(float(z.mean())) < 0.03 and abs(float(z.std()) - 1.0) < 0.03
