"""Parity of the CUDA path with the CPU oracle, through the C ABI (ctypes binding) and the
Python API.  Integer results (ids, counts, graphs, file bytes) must be bit-exact; distances
are bit-exact too because both sides use the same fp32 summation order, and additionally
within 1e-5 relative of a float64 recomputation."""
import json
import os

import numpy as np
import pytest

import oracle
from oracle import index_file
from conftest import assert_same_bits, engine_options, small_workload
from cuhnsw_b200 import CuHNSW
from cuhnsw_b200 import datasets as ds

pytestmark = pytest.mark.gpu


def engine_from_oracle_graph(g, opt, tmp_path, labels=None, **extra):
  path = str(tmp_path / "g.index")
  index_file.save(path, g, opt.get("level_mult", 0.3), opt.get("ef_construction", 100), labels=labels)
  eng = CuHNSW(engine_options(opt, **extra))
  eng.load_index(path)
  return eng


# ---------------------------------------------------------------- distance
@pytest.mark.parametrize("d", [1, 3, 4, 31, 33, 50, 64, 96, 128, 129, 500, 960, 1000])
@pytest.mark.parametrize("dist_type", ["dot", "l2"])
def test_distance_bit_exact(d, dist_type):
  rng = np.random.default_rng(1000 + d)
  base = rng.standard_normal((257, d)).astype(np.float32)
  eng = CuHNSW(engine_options({"dist_type": dist_type}))
  eng.set_data(base)
  src = rng.integers(0, len(base), 600).astype(np.int32)
  dst = rng.integers(0, len(base), 600).astype(np.int32)
  got = eng.obj.batch_distance(src, dst)
  want = np.array([oracle.distance(base[a], base[b], dist_type) for a, b in zip(src, dst)], np.float32)
  assert_same_bits(got, want)
  a, b = base[src].astype(np.float64), base[dst].astype(np.float64)
  exact = -(a * b).sum(1) if dist_type == "dot" else ((a - b) ** 2).sum(1)
  scale = np.abs(a * b).sum(1) if dist_type == "dot" else np.abs(exact)
  assert (np.abs(got - exact) <= 1e-5 * np.maximum(scale, 1e-30)).all()
  with pytest.raises(RuntimeError, match="out of range"):
    eng.obj.batch_distance(np.array([0], np.int32), np.array([len(base)], np.int32))


# ---------------------------------------------------------------- search
SEARCH_CASES = [  # workload, n, nq, ef list
  ("angular_toy", 20000, 500, (10, 50, 300)),
  ("angular_full", 30000, 300, (50, 100, 200, 300)),
  ("l2_integer", 10000, 300, (64, 128, 256)),
  ("highdim_l2", 3000, 100, (100, 300, 500)),
  ("sharded_100m", 10000, 300, (128,)),
]


@pytest.mark.parametrize("name,n,nq,efs", SEARCH_CASES)
def test_search_ids_and_distances_bit_exact(name, n, nq, efs, tmp_path):
  base, q, opt = small_workload(name, n, nq)
  levels = ds.random_levels(n, opt["seed"], opt["level_mult"])
  g = oracle.build_graph(base, levels, opt["max_m"], opt["max_m0"], opt["dist_type"], opt["ef_construction"],
                         bmax=512)
  eng = engine_from_oracle_graph(g, opt, tmp_path)
  truth = ds.ground_truth(base, q, 10, opt["dist_type"])
  for ef in efs:
    ids, dist, found = eng.search_knn(q, 10, ef)
    oids, odist, ofound = oracle.search(g, q, 10, ef)
    assert (ids == oids).all(), f"{name} ef={ef}"
    assert (found == ofound).all()
    assert_same_bits(dist, odist)
    # float64 recomputation, tolerance 1e-5 relative
    sel = base[ids[:, 0]].astype(np.float64)
    qq = q.astype(np.float64)
    exact = -(sel * qq).sum(1) if opt["dist_type"] == "dot" else ((sel - qq) ** 2).sum(1)
    scale = np.abs(sel * qq).sum(1) if opt["dist_type"] == "dot" else np.abs(exact)
    assert (np.abs(dist[:, 0] - exact) <= 1e-5 * np.maximum(scale, 1e-30)).all()
  assert ds.recall(ids, truth) > 0.9


@pytest.mark.parametrize("d,dist_type", [(960, "l2"), (200, "dot"), (129, "l2")])
def test_wide_rows_every_search_kernel_gives_the_oracle_answer(d, dist_type, tmp_path):
  """Rows wider than 128 floats have three kernels: a CTA of four warps per query, a warp per query with
  deep load batches (few queries), a warp per query with shallow batches (many queries)."""
  rng = np.random.default_rng(d)
  n, nq = 3000, 120
  base = rng.standard_normal((n, d)).astype(np.float32)
  q = rng.standard_normal((nq, d)).astype(np.float32)
  opt = {"dist_type": dist_type, "max_m": 12, "max_m0": 24, "ef_construction": 100, "level_mult": 0.4, "seed": 5}
  levels = ds.random_levels(n, opt["seed"], opt["level_mult"])
  g = oracle.build_graph(base, levels, 12, 24, dist_type, 100, bmax=512)
  # ef 1500: lists long enough for the CTA-per-query kernel to move their keys with all four warps
  want = {ef: oracle.search(g, q, 10, ef) for ef in (10, 100, 400, 1500)}
  for team in (1, 0, -1):
    eng = engine_from_oracle_graph(g, opt, tmp_path, search_team=team)
    for ef, (oids, odist, ofound) in want.items():
      ids, dist, found = eng.search_knn(q, 10, ef)
      assert (ids == oids).all() and (found == ofound).all(), f"team={team} ef={ef}"
      assert_same_bits(dist, odist)
    # 15 copies of the batch: more queries than ten per SM, the many-queries kernel (team = 0, -1)
    ids, dist, found = eng.search_knn(np.tile(q, (15, 1)), 10, 100)
    assert (ids == np.tile(want[100][0], (15, 1))).all()
    assert_same_bits(dist, np.tile(want[100][1], (15, 1)))


@pytest.mark.parametrize("name,n,team", [("angular_toy", 20000, -1), ("highdim_l2", 3000, 1), ("highdim_l2", 3000, 0)])
def test_batches_of_several_waves_are_served_longest_first_with_the_same_answers(name, n, team, tmp_path):
  """More queries than resident warps: the engine first descends the upper layers for every query, sorts the
  queries by the distance of the entry it found and serves the farthest first.  Answers must not change."""
  base, q, opt = small_workload(name, n, 700)
  levels = ds.random_levels(n, opt["seed"], opt["level_mult"])
  g = oracle.build_graph(base, levels, opt["max_m"], opt["max_m0"], opt["dist_type"], opt["ef_construction"],
                         bmax=512)
  oids, odist, ofound = oracle.search(g, q, 10, 40)
  expansions = int(oracle.search(g, q, 10, 40, counters=True)[3][:, 1].sum())
  # 5600 queries: more than 32 warps on each of 148 SMs, ordered by the single-CTA sort; 21 000: beyond that
  # sort's reach, ordered by the device-wide radix sort
  for reps in (8, 30) if team < 0 else (8,):
    big = np.tile(q, (reps, 1))
    for schedule in (True, False):
      eng = engine_from_oracle_graph(g, opt, tmp_path, search_team=team, search_schedule=schedule)
      eng.obj.enable_stats(True)
      ids, dist, found = eng.search_knn(big, 10, 40)
      stats = eng.obj.get_stats()
      assert (ids == np.tile(oids, (reps, 1))).all() and (found == np.tile(ofound, reps)).all(), f"schedule={schedule}"
      assert_same_bits(dist, np.tile(odist, (reps, 1)))
      assert stats["expansions"] == reps * expansions


def test_search_equals_reference_kernels_on_their_golden_vectors(golden_dir):
  """The reference's own LoadIndex + SearchGraph output on the same file, queries and ef."""
  z = np.load(os.path.join(golden_dir, "ref_search_angular.npz"))
  eng = CuHNSW(engine_options({"dist_type": "dot"}))
  eng.load_index(os.path.join(golden_dir, "ref_search_angular.index"))
  for ef in (10, 40, 120):
    ids, dist, found = eng.search_knn(z["queries"], 10, ef)
    assert (ids == z[f"ids_ef{ef}"]).all() and (found == z[f"found_ef{ef}"]).all()
    np.testing.assert_allclose(dist, z[f"dist_ef{ef}"], rtol=1e-5, atol=1e-6)
  z = np.load(os.path.join(golden_dir, "ref_built_angular.npz"))
  eng = CuHNSW(engine_options({"dist_type": "dot"}))
  eng.load_index(os.path.join(golden_dir, "ref_built_angular.index"))
  ids, dist, found = eng.search_knn(z["queries"], 10, 40)
  assert (ids == z["ids_ef40"]).all()
  np.testing.assert_allclose(dist, z["dist_ef40"], rtol=1e-5, atol=1e-6)


def test_exact_ties_are_broken_by_id(golden_dir, tmp_path):
  z = np.load(os.path.join(golden_dir, "ref_search_ties.npz"))
  g = index_file.load(os.path.join(golden_dir, "ref_search_ties.index"), "l2")
  eng = CuHNSW(engine_options({"dist_type": "l2"}))
  eng.load_index(os.path.join(golden_dir, "ref_search_ties.index"))
  for ef in (10, 40, 120):
    ids, dist, found = eng.search_knn(z["queries"], 10, ef)
    oids, odist, _ = oracle.search(g, z["queries"], 10, ef)
    assert (ids == oids).all()
    assert_same_bits(dist, odist)
  np.testing.assert_array_equal(dist, z["dist_ef120"])  # equals the reference's distance rows at a wide beam


def test_search_edge_cases(tmp_path):
  base, q, opt = small_workload("angular_toy", 3000, 64)
  levels = ds.random_levels(len(base), 777, opt["level_mult"])
  g = oracle.build_graph(base, levels, 12, 24, "dot", 60, bmax=64)
  labels = np.arange(len(base))[::-1] * 3 + 7  # ids are mapped through the file's labels after load_index
  eng = engine_from_oracle_graph(g, opt, tmp_path, labels=labels)
  ids, dist, found = eng.search_knn(q, 10, 40)
  oids, odist, _ = oracle.search(g, q, 10, 40)
  assert (ids == labels[oids]).all()
  # ef_search below topk is raised to topk (cuhnsw/pyhnsw.py:80)
  a = eng.search_knn(q, 10, 1)
  b = eng.search_knn(q, 10, 10)
  assert all((x == y).all() for x, y in zip(a, b))
  # one query given as a 1-d array (cuhnsw/bindings.cc:62-64)
  one = eng.search_knn(q[0], 10, 40)
  assert one[0].shape == (1, 10) and (one[0][0] == ids[0]).all()
  # topk and ef larger than the index: short rows, found < topk, exact answer
  tiny = oracle.build_graph(base[:7], np.zeros(7, np.int32), 12, 24, "dot", 30)
  te = engine_from_oracle_graph(tiny, opt, tmp_path)
  ids, dist, found = te.search_knn(q[:9], 16, 64)
  bi, _ = oracle.bruteforce(base[:7], q[:9], 7, "dot")
  assert (found == 7).all() and (ids[:, :7] == bi).all() and (ids[:, 7:] == -1).all() and np.isinf(dist[:, 7:]).all()
  # large topk / ef
  ids, dist, found = eng.search_knn(q[:16], 100, 1000)
  oids, odist, ofound = oracle.search(g, q[:16], 100, 1000)
  assert (labels[oids] == ids).all() and (found == ofound).all()
  # zero queries
  ids, dist, found = eng.search_knn(np.zeros((0, 50), np.float32), 10, 40)
  assert ids.shape == (0, 10)
  with pytest.raises(RuntimeError, match="8192"):
    eng.search_knn(q[:2], 10, 10000)
  # queries narrower or wider than the index are refused before the engine reads them
  for bad in (np.zeros((2, 49), np.float32), np.zeros(51, np.float32)):
    with pytest.raises(RuntimeError, match="dimensions"):
      eng.search_knn(bad, 10, 40)
    with pytest.raises(RuntimeError, match="dimensions"):
      eng.obj.search_knn_noalloc(bad, 10, 40, np.zeros((2, 10), np.int32), np.zeros((2, 10), np.float32),
                                 np.zeros(2, np.int32))


def test_user_visited_table_size_does_not_change_results(tmp_path):
  """The visited table may forget (never invent) ids: any size gives the same answer."""
  base, q, opt = small_workload("angular_toy", 20000, 200)
  levels = ds.random_levels(len(base), 777, opt["level_mult"])
  g = oracle.build_graph(base, levels, 12, 24, "dot", 110, bmax=512)
  want = oracle.search(g, q, 10, 300)[0]
  for size in (64, 256, 4096):
    eng = engine_from_oracle_graph(g, opt, tmp_path, visited_table_size=size)
    assert (eng.search_knn(q, 10, 300)[0] == want).all()


def test_reverse_cand_search_and_build_bit_exact(tmp_path):
  """reverse_cand=True expands the farthest unexpanded candidate first, in search and in build
  (cuda_utils_kernels.cuh:113-124, cuhnsw_build.cu:176,270)."""
  base, q, opt = small_workload("angular_toy", 6000, 200)
  eng = CuHNSW(engine_options(opt, reverse_cand=True, batch_max=400))
  eng.set_data(base)
  eng.build()
  levels, rows0, rows_u = eng.obj.get_graph()
  g = oracle.build_graph(base, levels, 12, 24, "dot", 110, bmax=400, reverse_cand=True)
  assert (rows0 == g.rows0).all() and (rows_u[:g.rowsU.shape[0]] == g.rowsU).all()
  for ef in (10, 64, 200):
    ids, dist, found = eng.search_knn(q, 10, ef)
    oids, odist, ofound = oracle.search(g, q, 10, ef, reverse_cand=True)
    assert (ids == oids).all() and (found == ofound).all()
    assert_same_bits(dist, odist)
  # the forward search on the same graph is a different walk
  fwd = CuHNSW(engine_options(opt))
  path = str(tmp_path / "r.index")
  eng.save_index(path)
  fwd.load_index(path)
  assert (fwd.search_knn(q, 10, 64)[0] == oracle.search(g, q, 10, 64)[0]).all()


# ---------------------------------------------------------------- build
BUILD_CASES = [  # workload, n, heuristic_coef, save_remains, batch_max
  ("angular_toy", 20000, 0.25, False, 0),
  ("angular_toy", 6000, 0.0, False, 100),
  ("angular_toy", 6000, 0.0, True, 777),
  ("angular_toy", 3000, 1.0, False, 1),
  ("l2_integer", 8000, 0.25, False, 0),
  ("highdim_l2", 2500, 0.25, False, 300),
  ("sharded_100m", 8000, 0.25, True, 1000),
]


@pytest.mark.parametrize("name,n,coef,save_remains,batch_max", BUILD_CASES)
def test_built_graph_bit_exact_with_oracle_on_the_same_batch_schedule(name, n, coef, save_remains, batch_max):
  base, q, opt = small_workload(name, n, 200)
  eopt = engine_options(opt, heuristic_coef=coef, save_remains=save_remains)
  if batch_max:
    eopt["batch_max"] = batch_max
  eng = CuHNSW(eopt)
  eng.set_data(base)
  eng.build()
  info = eng.obj.describe()
  levels, rows0, rows_u = eng.obj.get_graph()
  assert (levels == ds.random_levels(n, opt["seed"], opt["level_mult"])).all()
  bmax = batch_max or int(4 * 10 * (info["sm_count"] * 128 // 32))
  g = oracle.build_graph(base, levels, opt["max_m"], opt["max_m0"], opt["dist_type"], opt["ef_construction"], coef,
                         save_remains, bmax=bmax, ramp_div=4)
  assert info["max_level"] == g.max_level and info["enter_point"] == g.enter_point
  assert (rows0 == g.rows0).all()
  assert (rows_u[:g.rowsU.shape[0]] == g.rowsU).all()
  ids, dist, _ = eng.search_knn(q, 10, 100)
  oids, odist, _ = oracle.search(g, q, 10, 100)
  assert (ids == oids).all()
  assert_same_bits(dist, odist)


@pytest.mark.parametrize("d,max_m,max_m0,efc,dist_type", [(7, 20, 40, 60, "l2"), (33, 32, 64, 100, "dot"),
                                                          (130, 5, 9, 300, "l2"), (1, 4, 8, 30, "l2")])
def test_unusual_shapes_build_and_search_bit_exact(d, max_m, max_m0, efc, dist_type):
  """Rows wider than one warp (max_m0 > 32), link budgets that are not multiples of 8, odd dimensions."""
  rng = np.random.default_rng(d * 1000 + max_m0)
  n = 3000
  base = rng.standard_normal((n, d)).astype(np.float32)
  q = rng.standard_normal((150, d)).astype(np.float32)
  opt = dict(dist_type=dist_type, max_m=max_m, max_m0=max_m0, ef_construction=efc, seed=5, batch_max=200)
  eng = CuHNSW(engine_options(opt))
  eng.set_data(base)
  eng.build()
  levels, rows0, rows_u = eng.obj.get_graph()
  assert (levels == ds.random_levels(n, 5, 1 / np.log(max_m))).all()  # level_mult defaults to 1 / ln(max_m)
  g = oracle.build_graph(base, levels, max_m, max_m0, dist_type, efc, 0.25, False, bmax=200)
  assert (rows0 == g.rows0).all() and (rows_u[:g.rowsU.shape[0]] == g.rowsU).all()
  for ef in (10, 90):
    ids, dist, found = eng.search_knn(q, 10, ef)
    oids, odist, ofound = oracle.search(g, q, 10, ef)
    assert (ids == oids).all() and (found == ofound).all()
    assert_same_bits(dist, odist)


def test_build_quality_not_below_reference_kernels(golden_dir):
  """recall@10 on the 100 000-point workload vs what the reference's own build reached with the
  same options on a B200 (tests/golden/ref_quality.json), tolerance 0.005; and vs the oracle's
  strictly sequential build."""
  ref = json.load(open(os.path.join(golden_dir, "ref_quality.json")))
  base, q, spec = ds.make("angular_toy", nq=2000)
  opt = dict(spec["opt"], nrz=False)
  eng = CuHNSW(engine_options(opt))
  eng.set_data(base)
  eng.build()
  truth = ds.ground_truth(base, q, 10, "dot", device="cuda")
  levels = ds.random_levels(len(base), 777, opt["level_mult"])
  seq = oracle.build_graph(base, levels, 12, 24, "dot", 110, bmax=1)
  for ef in (50, 100, 300):
    rec = ds.recall(eng.search_knn(q, 10, ef)[0], truth)
    assert rec >= ref["recall_at_10"][str(ef)] - 0.005, (ef, rec)
    assert rec >= ds.recall(oracle.search(seq, q, 10, ef)[0], truth) - 0.005, (ef, rec)


def test_degenerate_builds():
  # a single level, one node, two nodes, duplicates of one point
  for n in (1, 2, 5):
    base = np.random.default_rng(n).standard_normal((n, 20)).astype(np.float32)
    eng = CuHNSW(engine_options({"dist_type": "l2", "level_mult": 1e-9}))
    eng.set_data(base)
    eng.build()
    ids, dist, found = eng.search_knn(base, min(n, 3), 10)
    assert (found == min(n, 3)).all() and (ids[:, 0] == np.arange(n)).all() and (dist[:, 0] == 0).all()
  base = np.ones((300, 8), np.float32)
  eng = CuHNSW(engine_options({"dist_type": "l2"}))
  eng.set_data(base)
  eng.build()
  levels, rows0, rows_u = eng.obj.get_graph()
  g = oracle.build_graph(base, levels, 12, 24, "l2", 150, bmax=int(4 * 10 * eng.obj.describe()["sm_count"] * 4))
  assert (rows0 == g.rows0).all()
  ids, dist, found = eng.search_knn(base[:4], 10, 50)
  assert (dist == 0).all() and (ids == oracle.search(g, base[:4], 10, 50)[0]).all()


# ---------------------------------------------------------------- fp16 rows
def _rounded(x, row_dtype="f16"):
  if row_dtype == "bf16":
    import torch
    return torch.from_numpy(np.ascontiguousarray(x)).to(torch.bfloat16).to(torch.float32).numpy()
  return x.astype(np.float16).astype(np.float32)


@pytest.mark.parametrize("d,dist_type,row_dtype", [(50, "dot", "f16"), (33, "l2", "f16"), (128, "l2", "f16"),
                                                   (200, "dot", "f16"), (960, "l2", "f16"), (50, "dot", "bf16"),
                                                   (97, "l2", "bf16"), (960, "l2", "bf16")])
def test_half_rows_give_the_canonical_distance_over_the_rounded_values(d, dist_type, row_dtype, tmp_path):
  """row_dtype = f16 / bf16 stores round-to-nearest-even 16-bit values; every distance, and therefore every
  search and every built graph, equals the fp32 oracle run on the rounded vectors, bit for bit."""
  rng = np.random.default_rng(77 + d)
  n = 3000
  base = (rng.standard_normal((n, d)) * (3.0 if dist_type == "l2" else 1.0)).astype(np.float32)
  q = rng.standard_normal((150, d)).astype(np.float32)
  base_r = _rounded(base, row_dtype)
  opt = {"dist_type": dist_type, "max_m": 12, "max_m0": 24, "ef_construction": 80, "level_mult": 0.4, "seed": 9,
         "row_dtype": row_dtype, "batch_max": 300}
  eng = CuHNSW(engine_options(opt))
  eng.set_data(base)
  src = rng.integers(0, n, 500).astype(np.int32)
  dst = rng.integers(0, n, 500).astype(np.int32)
  got = eng.obj.batch_distance(src, dst)
  want = np.array([oracle.distance(base_r[a], base_r[b], dist_type) for a, b in zip(src, dst)], np.float32)
  assert_same_bits(got, want)
  # build: same graph as the oracle on the rounded rows with the same batch schedule
  eng.build()
  levels, rows0, rows_u = eng.obj.get_graph()
  g = oracle.build_graph(base_r, levels, 12, 24, dist_type, 80, bmax=300)
  assert (rows0 == g.rows0).all() and (rows_u[:g.rowsU.shape[0]] == g.rowsU).all()
  # search: fp32 queries against half rows
  for ef in (10, 100):
    ids, dist, found = eng.search_knn(q, 10, ef)
    oids, odist, ofound = oracle.search(g, q, 10, ef)
    assert (ids == oids).all() and (found == ofound).all()
    assert_same_bits(dist, odist)
  # the file holds the rounded values as fp32; loading it into half rows loses nothing
  p1, p2 = str(tmp_path / "h1.index"), str(tmp_path / "h2.index")
  eng.save_index(p1)
  assert (index_file.load(p1, dist_type).vec == base_r).all()
  eng2 = CuHNSW(engine_options({"dist_type": dist_type, "row_dtype": row_dtype}))
  eng2.load_index(p1)
  eng2.save_index(p2)
  assert open(p1, "rb").read() == open(p2, "rb").read()
  a, b = eng.search_knn(q, 10, 50), eng2.search_knn(q, 10, 50)
  assert all((x == y).all() for x, y in zip(a, b))


def test_half_rows_degenerate_shapes():
  """One dimension, one row, empty index, values that overflow or underflow half precision."""
  rng = np.random.default_rng(3)
  for n, d in ((1, 1), (5, 3), (40, 17)):
    base = rng.standard_normal((n, d)).astype(np.float32)
    base[0, 0] = 1e-6   # subnormal in half
    if n > 1:
      base[1, 0] = 7e4  # beyond the largest half: stored as +inf, like numpy's conversion
    eng = CuHNSW(engine_options({"dist_type": "l2", "row_dtype": "f16", "max_m": 4, "max_m0": 8, "ef_construction": 16}))
    eng.set_data(base)
    eng.build()
    levels, rows0, _ = eng.obj.get_graph()
    with np.errstate(over="ignore"):
      g = oracle.build_graph(_rounded(base), levels, 4, 8, "l2", 16, bmax=int(4 * 10 * eng.obj.describe()["sm_count"] * 4))
      assert (rows0 == g.rows0).all()
      q = rng.standard_normal((6, d)).astype(np.float32)
      ids, dist, found = eng.search_knn(q, 4, 16)
      oids, odist, ofound = oracle.search(g, q, 4, 16)
    assert (ids == oids).all() and (found == ofound).all()
    assert_same_bits(dist, odist)
  empty = CuHNSW(engine_options({"dist_type": "l2", "row_dtype": "f16"}))
  empty.set_data(np.zeros((0, 8), np.float32))
  empty.build()
  ids, dist, found = empty.search_knn(np.zeros((3, 8), np.float32), 5, 10)
  assert (found == 0).all() and (ids == -1).all()
  # empty slots read +inf, bit for bit, from every entry point
  inf_bits = np.full((3, 5), 0x7f800000, np.uint32)
  assert (dist.view(np.uint32) == inf_bits).all()
  out = (np.zeros((3, 5), np.int32), np.zeros((3, 5), np.float32), np.ones(3, np.int32))
  empty.obj.search_knn_noalloc(np.zeros((3, 8), np.float32), 5, 10, *out)
  assert (out[1].view(np.uint32) == inf_bits).all() and (out[0] == -1).all() and (out[2] == 0).all()
  import torch
  dev = [torch.zeros((3, 8), device="cuda"), torch.zeros((3, 5), dtype=torch.int32, device="cuda"),
         torch.zeros((3, 5), device="cuda"), torch.ones(3, dtype=torch.int32, device="cuda")]
  empty.obj.search_knn_device(dev[0].data_ptr(), 3, 5, 10, dev[1].data_ptr(), dev[2].data_ptr(), dev[3].data_ptr())
  empty.obj.synchronize()
  assert (dev[2].cpu().numpy().view(np.uint32) == inf_bits).all() and (dev[1].cpu().numpy() == -1).all()


def test_half_rows_keep_recall():
  base, q, opt = small_workload("angular_full", 50000, 500)
  truth = ds.ground_truth(base, q, 10, opt["dist_type"])
  rec = {}
  for dt in ("f32", "f16"):
    eng = CuHNSW(engine_options(opt, row_dtype=dt))
    eng.set_data(base)
    eng.build()
    rec[dt] = ds.recall(eng.search_knn(q, 10, 200)[0], truth)
  assert rec["f16"] >= rec["f32"] - 0.01, rec
  with pytest.raises(RuntimeError, match="row_dtype"):
    CuHNSW(engine_options(opt, row_dtype="f8"))


# ---------------------------------------------------------------- index file
def test_save_load_save_is_byte_identical_and_oracle_readable(tmp_path):
  base, q, opt = small_workload("angular_toy", 5000, 100)
  eng = CuHNSW(engine_options(opt, batch_max=256))
  eng.set_data(base)
  eng.build()
  p1, p2 = str(tmp_path / "a.index"), str(tmp_path / "b.index")
  eng.save_index(p1)
  levels, rows0, rows_u = eng.obj.get_graph()
  g = index_file.load(p1, "dot")  # independent numpy reader
  assert (g.vec == base).all() and (g.rows0 == rows0).all() and (g.levels == levels).all()
  assert (g.rowsU == rows_u[:g.rowsU.shape[0]]).all() and (g.labels == np.arange(len(base))).all()
  assert g.header["maxM"] == 12 and g.header["maxM0"] == 24 and g.header["ef_construction"] == 110
  assert g.header["mult"] == pytest.approx(opt["level_mult"])
  eng2 = CuHNSW(engine_options({"dist_type": "dot"}))
  eng2.load_index(p1)
  eng2.save_index(p2)  # the reference cannot do this (its load leaves levels off by one)
  assert open(p1, "rb").read() == open(p2, "rb").read()
  a, b = eng.search_knn(q, 10, 64), eng2.search_knn(q, 10, 64)
  assert all((x == y).all() for x, y in zip(a, b))


@pytest.mark.parametrize("n,d,max_m,max_m0", [(1, 1, 2, 2), (3, 5, 4, 9), (700, 257, 32, 64), (2000, 50, 12, 24)])
def test_files_of_odd_shapes_and_64_bit_labels_round_trip(n, d, max_m, max_m0, tmp_path):
  """save_index puts the records together on the device: one row, link budgets that are not multiples of 8 or
  fill two warps, rows wider than 128 floats; and labels beyond 32 bits, which only the host holds."""
  rng = np.random.default_rng(n + d)
  base = rng.standard_normal((n, d)).astype(np.float32)
  opt = dict(dist_type="l2", max_m=max_m, max_m0=max_m0, ef_construction=max(max_m0, 40), seed=9)
  eng = CuHNSW(engine_options(opt))
  eng.set_data(base)
  eng.build()
  p1, p2, p3 = (str(tmp_path / f"{k}.index") for k in "abc")
  eng.save_index(p1)
  levels, rows0, rows_u = eng.obj.get_graph()
  g = index_file.load(p1, "l2")
  assert (g.vec == base).all() and (g.rows0 == rows0).all() and (g.levels == levels).all()
  assert (g.rowsU == rows_u[:g.rowsU.shape[0]]).all() and (g.labels == np.arange(n)).all()
  # the same index as the numpy writer lays it out, with labels that need all 64 bits
  labels = np.arange(n, dtype=np.int64) * (1 << 33) + 7
  index_file.save(p2, g, g.header["mult"], g.header["ef_construction"], labels=labels)
  eng2 = CuHNSW(engine_options({"dist_type": "l2"}))
  eng2.load_index(p2)
  eng2.save_index(p3)
  assert open(p2, "rb").read() == open(p3, "rb").read()


def test_file_written_by_reference_round_trips(golden_dir, tmp_path):
  src = os.path.join(golden_dir, "ref_built_angular.index")
  eng = CuHNSW(engine_options({"dist_type": "dot"}))
  eng.load_index(src)
  out = str(tmp_path / "again.index")
  eng.save_index(out)
  a, b = index_file.load(src, "dot"), index_file.load(out, "dot")
  assert a.header == b.header
  assert (a.rows0 == b.rows0).all() and (a.rowsU == b.rowsU).all() and (a.vec == b.vec).all()
  assert (a.levels == b.levels).all() and (a.labels == b.labels).all()


# ---------------------------------------------------------------- device-pointer path, stats, merge
def test_device_pointer_search_and_counters(tmp_path):
  import torch
  base, q, opt = small_workload("angular_toy", 20000, 1000)
  eng = CuHNSW(engine_options(opt))
  eng.set_data(base)
  eng.build()
  host = eng.search_knn(q, 10, 100)
  qd = torch.from_numpy(q).cuda()
  ids = torch.empty((len(q), 10), dtype=torch.int32, device="cuda")
  dist = torch.empty((len(q), 10), dtype=torch.float32, device="cuda")
  found = torch.empty((len(q),), dtype=torch.int32, device="cuda")
  stream = torch.cuda.Stream()
  eng.obj.set_stream(stream.cuda_stream)
  eng.obj.enable_stats(True)
  eng.obj.search_knn_device(qd.data_ptr(), len(q), 10, 100, ids.data_ptr(), dist.data_ptr(), found.data_ptr())
  eng.obj.synchronize()
  st = eng.obj.get_stats()
  assert (ids.cpu().numpy() == host[0]).all() and (found.cpu().numpy() == host[2]).all()
  assert_same_bits(dist.cpu().numpy(), host[1])
  levels, rows0, rows_u = eng.obj.get_graph()
  g = oracle.Graph(base, levels, 12, 24, "dot")
  g.rows0[:], g.deg0[:] = rows0, (rows0 >= 0).sum(1)
  g.rowsU[:], g.degU[:] = rows_u[:g.rowsU.shape[0]], (rows_u[:g.rowsU.shape[0]] >= 0).sum(1)
  _, _, _, cnt = oracle.search(g, q, 10, 100, counters=True)
  # expansions are deterministic; evaluations may repeat (lossy visited table) but never fall short
  assert st["expansions"] == int(cnt[:, 1].sum())
  assert st["sweeps"] == int(cnt[:, 2].sum())
  assert int(cnt[:, 0].sum()) <= st["evals"] <= 1.5 * int(cnt[:, 0].sum())
  eng.obj.set_stream(0)


def test_sharded_search_with_device_merge_equals_exact_answer():
  import torch
  from cuhnsw_b200 import multi
  base, q, opt = small_workload("sharded_100m", 12000, 300)
  parts = 4
  ids_blocks, dist_blocks = [], []
  qd = torch.from_numpy(q).cuda()
  for r in range(parts):
    lo, hi = multi.split_range(len(base), parts, r)
    eng = CuHNSW(engine_options(opt, batch_max=500))
    eng.set_data(base[lo:hi])
    eng.build()
    ids = torch.empty((len(q), 10), dtype=torch.int32, device="cuda")
    dist = torch.empty((len(q), 10), dtype=torch.float32, device="cuda")
    found = torch.empty((len(q),), dtype=torch.int32, device="cuda")
    eng.obj.search_knn_device(qd.data_ptr(), len(q), 10, hi - lo, ids.data_ptr(), dist.data_ptr(), found.data_ptr())
    eng.obj.synchronize()
    ids_blocks.append(torch.where(ids >= 0, ids + lo, ids))
    dist_blocks.append(dist)
  out_ids, out_d, found = multi.device_merge(torch.stack(ids_blocks), torch.stack(dist_blocks), 10)
  torch.cuda.synchronize()
  host_ids, host_d, host_found = multi.merge_topk_host(torch.stack(ids_blocks).cpu().numpy(),
                                                       torch.stack(dist_blocks).cpu().numpy(), 10)
  assert (out_ids.cpu().numpy() == host_ids).all() and (found.cpu().numpy() == host_found).all()
  assert_same_bits(out_d.cpu().numpy(), host_d)
  exact, _ = oracle.bruteforce(base, q, 10, "dot")
  assert (out_ids.cpu().numpy() == exact).all()  # ef = shard size makes every shard exact
  # the same merge reading the [parts, 2, nq, k] buffer an all-gather fills, shard-local ids + offsets
  from cuhnsw_b200.cuhnsw_bind import load_library
  local_ids = [torch.where(b >= 0, b - multi.split_range(len(base), parts, r)[0], b) for r, b in enumerate(ids_blocks)]
  gathered = torch.stack([torch.stack([i, d.view(torch.int32)]) for i, d in zip(local_ids, dist_blocks)]).contiguous()
  offsets = torch.tensor([multi.split_range(len(base), parts, r)[0] for r in range(parts)], dtype=torch.int32,
                         device="cuda")
  g_ids, g_d, g_found = torch.empty_like(out_ids), torch.empty_like(out_d), torch.empty_like(found)
  rc = load_library().cuhnsw_merge_topk_gathered_device(
    gathered.data_ptr(), offsets.data_ptr(), parts, len(q), 10, g_ids.data_ptr(), g_d.data_ptr(), g_found.data_ptr(),
    torch.cuda.current_stream().cuda_stream)
  torch.cuda.synchronize()
  assert rc == 0 and (g_ids == out_ids).all() and (g_found == found).all()
  assert_same_bits(g_d.cpu().numpy(), out_d.cpu().numpy())


# ---------------------------------------------------------------- full size, size-independent properties
def test_full_size_angular_properties():
  """N = 1 183 514: rows full, ascending, unique; distances equal a recomputation; recall target met."""
  import torch
  base, q, spec = ds.make("angular_full", nq=2000)
  opt = dict(spec["opt"], nrz=False)
  eng = CuHNSW(engine_options(opt))
  eng.set_data(base)
  eng.build()
  assert eng.obj.last_build_seconds() < 60
  ids, dist, found = eng.search_knn(q, 10, 300)
  assert (found == 10).all()
  assert (np.diff(dist, axis=1) >= 0).all()
  assert all(len(set(r.tolist())) == 10 for r in ids)
  assert ids.min() >= 0 and ids.max() < len(base)
  re = -(base[ids.reshape(-1)].astype(np.float64) * np.repeat(q, 10, 0).astype(np.float64)).sum(1).reshape(ids.shape)
  np.testing.assert_allclose(dist, re, rtol=1e-5, atol=1e-6)
  truth = ds.ground_truth(base, q, 10, "dot", device="cuda")
  assert ds.recall(ids, truth) >= 0.95
  # repeatable, and independent of how the batch is cut
  again = eng.search_knn(q, 10, 300)[0]
  assert (again == ids).all()
  assert (eng.search_knn(q[1000:1300], 10, 300)[0] == ids[1000:1300]).all()
  levels, rows0, _ = eng.obj.get_graph()
  deg = (rows0 >= 0).sum(1)
  assert deg.max() <= 24 and (rows0 != np.arange(len(base))[:, None]).all()
  assert (np.sort(np.where(rows0 >= 0, rows0, -1), axis=1)[:, 1:][(np.sort(rows0, axis=1)[:, 1:] >= 0)] !=
          np.sort(np.where(rows0 >= 0, rows0, -1), axis=1)[:, :-1][(np.sort(rows0, axis=1)[:, 1:] >= 0)]).all()
