"""Randomly drawn small configurations: index size from 1 row up, odd and wide dimensions, link budgets up to
64, every option of the neighbour selection (cuda_build_kernels.cuh:68-162 of the reference), reverse_cand
(cuda_utils_kernels.cuh:113-124), data with many exact ties or many duplicate points, 16-bit rows, query batches
from 1 to more than a wave, topk above ef.  The GPU's graph must equal the oracle's on the same batch schedule
and the searches must agree in ids, counts and distance bits."""
import numpy as np
import pytest

import oracle
from conftest import assert_same_bits, engine_options
from cuhnsw_b200 import CuHNSW

pytestmark = pytest.mark.gpu


def _stored(x, row_dtype):
  if row_dtype == "f16":
    return x.astype(np.float16).astype(np.float32)
  if row_dtype == "bf16":
    import torch
    return torch.from_numpy(x).to(torch.bfloat16).to(torch.float32).numpy()
  return x


def _draw(seed):
  rng = np.random.default_rng(seed)
  c = {"n": int(rng.choice([1, 2, 3, 17, 100, 700, 2500, 6000])),
       "d": int(rng.choice([1, 2, 3, 5, 8, 31, 32, 33, 50, 64, 65, 96, 100, 128, 129, 200, 257]))}
  c["max_m"] = int(rng.integers(2, 33))
  c["max_m0"] = int(rng.integers(c["max_m"], 65))
  c["efc"] = int(rng.integers(max(c["max_m0"], 8), 260))
  c["dist_type"] = str(rng.choice(["l2", "dot"]))
  c["coef"] = float(rng.choice([0.25, 0.0, 1.0, 0.6]))
  c["save_remains"] = bool(rng.integers(0, 2))
  c["reverse"] = bool(rng.integers(0, 4) == 0)
  c["level_mult"] = float(rng.choice([0.3, 0.5, 1.0 / np.log(max(c["max_m"], 2))]))
  c["batch_max"] = int(rng.choice([0, 0, 64, 500]))
  c["row_dtype"] = str(rng.choice(["f32", "f32", "f16", "bf16"]))
  kind = int(rng.integers(0, 3))
  n, d = c["n"], c["d"]
  if kind == 0:
    base = rng.standard_normal((n, d)).astype(np.float32)
  elif kind == 1:  # small integers: many exactly equal distances
    base = rng.integers(0, 3, (n, d)).astype(np.float32)
  else:  # copies of a few points: distance zero between neighbours
    few = max(1, n // 50)
    base = rng.standard_normal((few, d)).astype(np.float32)[rng.integers(0, few, n)]
  nq = int(rng.choice([1, 7, 150, 1200]))
  q = (rng.integers(0, 3, (nq, d)) if kind == 1 else rng.standard_normal((nq, d))).astype(np.float32)
  c["topk"] = int(rng.choice([1, 3, 10, 40]))
  c["ef"] = int(rng.choice([1, 10, 64, 200, 700, 3000]))  # 3000: lists whose places are searched span by span
  return c, base, q


@pytest.mark.parametrize("block", range(8))
def test_random_configurations_build_and_search_like_the_oracle(block):
  for seed in range(1000 + 12 * block, 1000 + 12 * (block + 1)):
    c, base, q = _draw(seed)
    opt = dict(dist_type=c["dist_type"], max_m=c["max_m"], max_m0=c["max_m0"], ef_construction=c["efc"],
               level_mult=c["level_mult"], seed=seed, heuristic_coef=c["coef"], save_remains=c["save_remains"],
               reverse_cand=c["reverse"], nrz=False, row_dtype=c["row_dtype"])
    if c["batch_max"]:
      opt["batch_max"] = c["batch_max"]
    eng = CuHNSW(engine_options(opt))
    eng.set_data(base)
    eng.build()
    info = eng.obj.describe()
    levels, rows0, rows_u = eng.obj.get_graph()
    bmax = c["batch_max"] or int(4 * 10 * (info["sm_count"] * 128 // 32))
    stored = _stored(base, c["row_dtype"])
    g = oracle.build_graph(stored, levels, c["max_m"], c["max_m0"], c["dist_type"], c["efc"], c["coef"],
                           c["save_remains"], bmax=bmax, ramp_div=4, reverse_cand=c["reverse"])
    what = f"seed {seed}: {c}"
    assert info["max_level"] == g.max_level and info["enter_point"] == g.enter_point, what
    assert (rows0 == g.rows0).all() and (rows_u[:g.rowsU.shape[0]] == g.rowsU).all(), what
    ids, dist, found = eng.search_knn(q, c["topk"], c["ef"])
    oids, odist, ofound = oracle.search(g, q, c["topk"], max(c["ef"], c["topk"]), reverse_cand=c["reverse"])
    assert (ids == oids).all() and (found == ofound).all(), what
    assert_same_bits(dist, odist)
