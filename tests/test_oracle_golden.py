"""Pins the CPU oracle: level draws produced by the reference's own Python code, and
search results / index files produced by the reference's own CUDA kernels on a B200
(tests/golden/make_level_draws.py, tests/golden/make_ref_fixtures.py)."""
import hashlib
import json
import os

import numpy as np
import pytest

import oracle
from oracle import index_file
from cuhnsw_b200 import datasets as ds


def test_level_draws_match_reference_python(golden_dir):
  cases = json.load(open(os.path.join(golden_dir, "level_draws.json")))
  assert len(cases) >= 6
  for c in cases:
    lv = ds.random_levels(c["num_data"], c["seed"], c["level_mult"])
    assert lv.dtype == np.int32
    assert hashlib.sha256(lv.tobytes()).hexdigest() == c["sha256"]
    assert [int(x) for x in lv[:64]] == c["first_64"]
    assert int(lv.max()) == c["max_level"]
    assert [int((lv >= l).sum()) for l in range(c["max_level"] + 1)] == c["nodes_per_level"]
    # enter point = first node that reaches the top level (cpp/src/cuhnsw_base.cu:134-141)
    assert int(np.argmax(lv == lv.max())) == c["enter_point"]


def test_level_known_answers_of_the_benchmark_sizes(golden_dir):
  cases = {(c["num_data"], round(c["level_mult"], 6)): c
           for c in json.load(open(os.path.join(golden_dir, "level_draws.json")))}
  c1 = cases[(100_000, round(1 / np.log(24), 6))]
  assert (c1["max_level"], c1["enter_point"], c1["nodes_per_level"]) == (3, 11619, [100000, 4254, 205, 13])
  c2 = cases[(1_183_514, round(1 / np.log(24), 6))]
  assert (c2["max_level"], c2["enter_point"], c2["nodes_per_level"]) == (4, 596640, [1183514, 49250, 2155, 90, 2])


@pytest.mark.parametrize("ef", [10, 40, 120])
def test_search_equals_reference_kernels_on_continuous_data(golden_dir, ef):
  """Same index file, same queries, same ef: ids bit-exact, distances within 1e-5 relative
  (the reference sums in a different fp32 order)."""
  z = np.load(os.path.join(golden_dir, "ref_search_angular.npz"))
  g = index_file.load(os.path.join(golden_dir, "ref_search_angular.index"), "dot")
  ids, dist, found = oracle.search(g, z["queries"], 10, ef)
  assert (ids == z[f"ids_ef{ef}"]).all()
  assert (found == z[f"found_ef{ef}"]).all()
  np.testing.assert_allclose(dist, z[f"dist_ef{ef}"], rtol=1e-5, atol=1e-6)


def test_search_on_tied_distances_agrees_up_to_tie_order(golden_dir):
  """Integer-valued vectors give many exactly equal distances.  The reference orders equal
  distances by heap position, the oracle by id, so only tie-independent facts are compared:
  every id the reference ranks strictly below its k-th distance is returned, and at a wide
  beam the distance rows are identical."""
  z = np.load(os.path.join(golden_dir, "ref_search_ties.npz"))
  g = index_file.load(os.path.join(golden_dir, "ref_search_ties.index"), "l2")
  ids, dist, found = oracle.search(g, z["queries"], 10, 120)
  rid, rdist = z["ids_ef120"], z["dist_ef120"]
  assert (found == z["found_ef120"]).all()
  np.testing.assert_array_equal(dist, rdist)  # sums of small integers are exact in fp32
  for a, b, db in zip(ids, rid, rdist):
    strict = set(b[db < db[-1]].tolist())
    assert strict <= set(a.tolist())
  # the oracle's own rule: ties ascending by id
  for a, da in zip(ids, dist):
    keys = list(zip(da.tolist(), a.tolist()))
    assert keys == sorted(keys)


def test_index_written_by_reference_build_loads_and_searches_identically(golden_dir):
  z = np.load(os.path.join(golden_dir, "ref_built_angular.npz"))
  g = index_file.load(os.path.join(golden_dir, "ref_built_angular.index"), "dot")
  h = g.header
  assert (h["cur_element_count"], h["maxM"], h["maxM0"], h["ef_construction"]) == (1200, 12, 24, 110)
  assert h["size_data_per_element"] == 4 + 4 * 24 + 4 * 50 + 8 and h["offsetData"] == 100 and h["label_offset"] == 300
  assert (g.levels == z["levels"]).all()  # link-list sizes encode the level of every node
  assert g.max_level == int(z["levels"].max()) and g.enter_point == int(np.argmax(z["levels"] == z["levels"].max()))
  assert (g.labels == np.arange(1200)).all()
  ids, dist, found = oracle.search(g, z["queries"], 10, 40)
  assert (ids == z["ids_ef40"]).all() and (found == z["found_ef40"]).all()
  np.testing.assert_allclose(dist, z["dist_ef40"], rtol=1e-5, atol=1e-6)


def test_oracle_build_quality_not_below_reference_kernels(golden_dir):
  """recall@10 of the oracle's builds on the 100 000-point workload vs the recall the reference's
  own build kernel reached on a B200 with the same options (tolerance 0.005)."""
  ref = json.load(open(os.path.join(golden_dir, "ref_quality.json")))
  base, q, spec = ds.make("angular_toy", nq=2000)
  opt = spec["opt"]
  assert len(base) == ref["n"]
  levels = ds.random_levels(len(base), opt["seed"], opt["level_mult"])
  truth = ds.ground_truth(base, q, 10, "dot")
  for bmax in (1, 23680):
    g = oracle.build_graph(base, levels, opt["max_m"], opt["max_m0"], "dot", opt["ef_construction"], 0.25, False,
                           bmax=bmax, ramp_div=4)
    for ef in (50, 100, 300):
      ids, _, _ = oracle.search(g, q, 10, ef)
      assert ds.recall(ids, truth) >= ref["recall_at_10"][str(ef)] - 0.005, (bmax, ef)
