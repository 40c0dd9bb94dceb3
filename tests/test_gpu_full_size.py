"""Parity with the CPU oracle at the sizes the benchmark is quoted on.

Walk lengths, the pressure on the visited table (16-bit tags at more than a million nodes) and the
scheduling of batches that need several waves all differ from the small slices of test_gpu_parity.py,
so the full configurations are built on the GPU, their graphs are handed to the oracle, and both sides
answer the same queries: ids and counts equal, distances bit-equal, and the device's count of expanded
rows equal to the oracle's (the walk itself is the same, not only its result)."""
import numpy as np
import pytest

import oracle
from conftest import assert_same_bits, engine_options, oracle_graph_of
from cuhnsw_b200 import CuHNSW
from cuhnsw_b200 import datasets as ds

pytestmark = pytest.mark.gpu


def check_against_oracle(name, nq, efs, variants, recall_floor):
  base, q, spec = ds.make(name, nq=nq)
  opt = dict(spec["opt"], nrz=False)
  g = None
  for extra in variants:
    eng = CuHNSW(engine_options(opt, **extra))
    eng.set_data(base)
    eng.build()
    if g is None:
      g = oracle_graph_of(eng, base, opt)
      want = {ef: oracle.search(g, q, 10, ef, counters=True) for ef in efs}
      truth = ds.ground_truth(base, q, 10, opt["dist_type"], device="cuda")
    else:
      # the build is deterministic: every variant holds the graph the oracle searches
      assert (eng.obj.get_graph()[1] == g.rows0).all()
    for ef in efs:
      oids, odist, ofound, cnt = want[ef]
      eng.obj.enable_stats(True)
      ids, dist, found = eng.search_knn(q, 10, ef)
      stats = eng.obj.get_stats()
      eng.obj.enable_stats(False)
      assert (ids == oids).all(), f"{name} ef={ef} {extra}"
      assert (found == ofound).all()
      assert_same_bits(dist, odist)
      assert stats["expansions"] == int(cnt[:, 1].sum()), f"{name} ef={ef} {extra}"
      assert stats["sweeps"] == int(cnt[:, 2].sum())
      assert stats["evals"] >= int(cnt[:, 0].sum())
    del eng
  assert ds.recall(want[max(efs)][0], truth) >= recall_floor


def test_angular_full_search_equals_oracle_at_full_size():
  """N = 1 183 514, d = 50: the headline configuration, at the two beam widths the benchmark can stop at,
  with the longest-first schedule on and off."""
  check_against_oracle("angular_full", 2500, (200, 300), ({"search_schedule": True}, {"search_schedule": False}), 0.95)


def test_l2_integer_search_equals_oracle_at_full_size():
  """N = 1 000 000, d = 128, integer coordinates: many exactly equal distances, broken by id."""
  check_against_oracle("l2_integer", 2000, (256,), ({},), 0.9)


def test_highdim_l2_search_equals_oracle_at_full_size():
  """N = 1 000 000, d = 960: the CTA-per-query kernel and the warp-per-query kernels on the same graph."""
  check_against_oracle("highdim_l2", 1000, (500,), ({"search_team": -1}, {"search_team": 1}, {"search_team": 0}), 0.9)
