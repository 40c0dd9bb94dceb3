"""Properties of the CPU oracle that do not need the reference: distance accuracy and
summation order, exactness of wide searches, determinism, neighbour-selection invariants,
index-file round trips."""
import os
import tempfile

import numpy as np
import pytest

import oracle
from oracle import index_file
from cuhnsw_b200 import datasets as ds


def canonical_numpy(a, b, dist_type):
  """Independent restatement of the fixed summation order (float64 emulation of fp32 fma)."""
  d = len(a)
  w = 32 if d <= 128 else 128
  acc = np.zeros(w, np.float32)
  for i in range(d):
    if dist_type == "dot":
      x, y = np.float64(a[i]), np.float64(b[i])
    else:
      x = y = np.float64(np.float32(a[i] - b[i]))
    acc[i % w] = np.float32(x * y + np.float64(acc[i % w]))
  lanes = [np.float32(np.float32(acc[4 * t] + acc[4 * t + 1]) + np.float32(acc[4 * t + 2] + acc[4 * t + 3]))
           for t in range(w // 4)]
  off = len(lanes) // 2
  while off:
    lanes = [np.float32(lanes[t] + lanes[t ^ off]) for t in range(len(lanes))]
    off //= 2
  return -lanes[0] if dist_type == "dot" else lanes[0]


@pytest.mark.parametrize("d", [1, 3, 4, 31, 32, 33, 50, 96, 128, 129, 960, 1000])
@pytest.mark.parametrize("dist_type", ["dot", "l2"])
def test_distance_order_and_accuracy(d, dist_type):
  rng = np.random.default_rng(d)
  for _ in range(6):
    a = rng.standard_normal(d).astype(np.float32)
    b = rng.standard_normal(d).astype(np.float32)
    got = np.float32(oracle.distance(a, b, dist_type))
    want = canonical_numpy(a, b, dist_type)
    # the float64 emulation of fma can differ by a double rounding: allow 1 ulp
    assert abs(float(got) - float(want)) <= float(np.spacing(np.abs(want))) + 0.0
    exact = -np.dot(a.astype(np.float64), b.astype(np.float64)) if dist_type == "dot" else \
      np.sum((a.astype(np.float64) - b.astype(np.float64)) ** 2)
    scale = np.sum(np.abs(a.astype(np.float64) * b.astype(np.float64))) if dist_type == "dot" else abs(exact)
    assert abs(float(got) - exact) <= 1e-5 * max(scale, 1e-30)
    assert oracle.distance(a, b, dist_type) == oracle.distance(b, a, dist_type)  # symmetric bit for bit


def test_integer_valued_l2_is_exact():
  rng = np.random.default_rng(0)
  a = rng.integers(0, 256, 128).astype(np.float32)
  b = rng.integers(0, 256, 128).astype(np.float32)
  assert oracle.distance(a, b, "l2") == float(np.sum((a.astype(np.int64) - b.astype(np.int64)) ** 2))


@pytest.fixture(scope="module")
def toy():
  base, q, spec = ds.make("angular_toy", n=3000, nq=200)
  opt = spec["opt"]
  levels = ds.random_levels(len(base), opt["seed"], opt["level_mult"])
  g = oracle.build_graph(base, levels, opt["max_m"], opt["max_m0"], "dot", opt["ef_construction"])
  return base, q, opt, levels, g


def test_wide_search_is_exact(toy):
  """With ef >= n every reachable node ends in the result set, so the answer is brute force."""
  base, q, _, _, g = toy
  ids, dist, found = oracle.search(g, q[:50], 10, len(base))
  bi, bd = oracle.bruteforce(base, q[:50], 10, "dot")
  assert (found == 10).all() and (ids == bi).all() and (dist == bd).all()


def test_rows_sorted_by_distance_then_id_and_unique(toy):
  _, q, _, _, g = toy
  ids, dist, found = oracle.search(g, q, 10, 40)
  for a, d, f in zip(ids, dist, found):
    keys = list(zip(d[:f].tolist(), a[:f].tolist()))
    assert keys == sorted(keys) and len(set(a[:f].tolist())) == f


def test_ef_is_raised_to_topk_and_short_rows(toy):
  base, q, opt, levels, g = toy
  a = oracle.search(g, q[:20], 10, 1)
  b = oracle.search(g, q[:20], 10, 10)
  assert all((x == y).all() for x, y in zip(a, b))
  tiny = oracle.build_graph(base[:5], np.zeros(5, np.int32), 12, 24, "dot", 50)
  ids, dist, found = oracle.search(tiny, q[:4], 10, 30)
  assert (found == 5).all() and (ids[:, 5:] == -1).all() and np.isinf(dist[:, 5:]).all()


def test_search_and_build_do_not_depend_on_thread_count(toy):
  base, q, opt, levels, g = toy
  r1 = oracle.search(g, q, 10, 64, nthreads=1)
  r4 = oracle.search(g, q, 10, 64, nthreads=4)
  assert all((x == y).all() for x, y in zip(r1, r4))
  for bmax in (1, 64):
    g1 = oracle.build_graph(base[:1500], levels[:1500], 12, 24, "dot", 60, bmax=bmax, nthreads=1)
    g4 = oracle.build_graph(base[:1500], levels[:1500], 12, 24, "dot", 60, bmax=bmax, nthreads=4)
    assert (g1.rows0 == g4.rows0).all() and (g1.rowsU == g4.rowsU).all()


@pytest.mark.parametrize("coef,save_remains", [(0.25, False), (0.0, False), (0.0, True), (1.0, False)])
def test_built_graph_invariants(coef, save_remains):
  base, q, spec = ds.make("l2_integer", n=1500, nq=50)
  opt = spec["opt"]
  levels = ds.random_levels(len(base), 777, opt["level_mult"])
  g = oracle.build_graph(base, levels, opt["max_m"], opt["max_m0"], "l2", 80, coef, save_remains, bmax=37)
  n = len(base)
  for rows, deg, cap in ((g.rows0, g.deg0, opt["max_m0"]), (g.rowsU[:int(levels.sum())], g.degU[:int(levels.sum())], opt["max_m"])):
    assert (deg <= cap).all() and (deg >= 0).all()
    for r, k in zip(rows, deg):
      live = r[:k]
      assert (live >= 0).all() and (live < n).all() and len(set(live.tolist())) == k and (r[k:] == -1).all()
  assert not (g.rows0 == np.arange(n)[:, None]).any()  # no self loops
  # upper-layer neighbours live on that layer
  for i in np.where(levels > 0)[0]:
    for l in range(levels[i]):
      row = g.rowsU[g.upper_base[i] + l]
      assert (levels[row[row >= 0]] >= l + 1).all()
  truth = ds.ground_truth(base, q, 10, "l2")
  ids, _, _ = oracle.search(g, q, 10, 100)
  assert ds.recall(ids, truth) > 0.9
  if save_remains:
    assert g.deg0.mean() > 0.9 * opt["max_m0"]


def test_sequential_and_batched_schedules_reach_similar_recall():
  base, q, spec = ds.make("angular_toy", n=20000, nq=500)
  opt = spec["opt"]
  levels = ds.random_levels(len(base), 777, opt["level_mult"])
  truth = ds.ground_truth(base, q, 10, "dot")
  rec = {}
  for bmax in (1, 23680):
    g = oracle.build_graph(base, levels, 12, 24, "dot", 110, bmax=bmax)
    rec[bmax] = ds.recall(oracle.search(g, q, 10, 50)[0], truth)
  assert rec[23680] >= rec[1] - 0.005, rec


def test_index_file_round_trip(toy):
  _, _, opt, levels, g = toy
  with tempfile.TemporaryDirectory() as tmp:
    p = os.path.join(tmp, "a.index")
    index_file.save(p, g, opt["level_mult"], opt["ef_construction"])
    assert os.path.getsize(p) == 96 + g.n * (4 + 4 * 24 + 4 * 50 + 8) + 4 * g.n + int(levels.sum()) * (4 + 4 * 12)
    g2 = index_file.load(p, "dot")
    assert (g2.rows0 == g.rows0).all() and (g2.deg0 == g.deg0).all() and (g2.vec == g.vec).all()
    assert (g2.levels == levels).all() and (g2.rowsU == g.rowsU).all()
    assert g2.enter_point == g.enter_point and g2.max_level == g.max_level
    assert g2.header["mult"] == opt["level_mult"]
