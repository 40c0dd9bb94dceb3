"""Cross-checks with hnswlib itself, the CPU library whose index files the reference reads and writes
(cpp/src/cuhnsw_base.cu:159-365; examples/example1.py:75-84,129-140 of the reference load a cuhnsw file into
hnswlib and the other way round).  hnswlib is not part of this environment: the module is skipped unless it can
be imported.  hnswlib sums its distances in its own SIMD order, so near-ties may fall either way: the comparison
is on the overlap of the answers, not on bits."""
import numpy as np
import pytest

from conftest import engine_options, small_workload
from cuhnsw_b200 import CuHNSW

hnswlib = pytest.importorskip("hnswlib")
pytestmark = pytest.mark.gpu


def _overlap(a, b):
  return float(np.mean([len(set(x) & set(y)) / len(x) for x, y in zip(a, b)]))


@pytest.mark.parametrize("name,space", [("angular_toy", "ip"), ("l2_integer", "l2")])
def test_index_built_here_searches_the_same_in_hnswlib(name, space, tmp_path):
  base, q, opt = small_workload(name, 20000, 500)
  eng = CuHNSW(engine_options(opt))
  eng.set_data(base)
  eng.build()
  path = str(tmp_path / "ours.index")
  eng.save_index(path)
  cpu = hnswlib.Index(space=space, dim=base.shape[1])
  cpu.load_index(path, max_elements=len(base))
  cpu.set_ef(100)
  labels, dist = cpu.knn_query(q, k=10)
  ids, ours, found = eng.search_knn(q, 10, 100)
  assert (found == 10).all()
  assert _overlap(ids, labels.astype(np.int64)) >= 0.98
  # hnswlib's inner-product space reports 1 - dot, this API -dot (cuda_dist_kernels.cuh:117 of the reference)
  theirs = np.sort(dist - 1.0 if space == "ip" else dist, axis=1)
  assert np.allclose(np.sort(ours, axis=1)[:, 0], theirs[:, 0], rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("name,space", [("angular_toy", "ip"), ("l2_integer", "l2")])
def test_index_built_by_hnswlib_loads_and_searches_here(name, space, tmp_path):
  base, q, opt = small_workload(name, 20000, 500)
  cpu = hnswlib.Index(space=space, dim=base.shape[1])
  cpu.init_index(max_elements=len(base), ef_construction=opt["ef_construction"], M=opt["max_m"], random_seed=7)
  cpu.add_items(base, np.arange(len(base)))
  path = str(tmp_path / "theirs.index")
  cpu.save_index(path)
  cpu.set_ef(100)
  labels, _ = cpu.knn_query(q, k=10)
  eng = CuHNSW(engine_options({"dist_type": opt["dist_type"]}))
  eng.load_index(path)
  ids, _, found = eng.search_knn(q, 10, 100)
  assert (found == 10).all()
  assert _overlap(ids, labels.astype(np.int64)) >= 0.98
  again = str(tmp_path / "again.index")
  eng.save_index(again)
  back = hnswlib.Index(space=space, dim=base.shape[1])
  back.load_index(again, max_elements=len(base))
  back.set_ef(100)
  assert _overlap(back.knn_query(q, k=10)[0], labels) >= 0.999
