import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
  sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
  config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def has_gpu():
  try:
    import torch
    return torch.cuda.is_available()
  except Exception:  # pylint: disable=broad-except
    return False


def pytest_collection_modifyitems(config, items):
  if has_gpu():
    return
  skip = pytest.mark.skip(reason="no CUDA device")
  for item in items:
    if "gpu" in item.keywords:
      item.add_marker(skip)


@pytest.fixture(scope="session")
def golden_dir():
  return GOLDEN


def small_workload(name, n, nq):
  """(base, queries, options) of a named workload at a reduced size."""
  from cuhnsw_b200 import datasets as ds
  base, q, spec = ds.make(name, n=n, nq=nq)
  opt = dict(spec["opt"])
  opt["nrz"] = False  # generators already normalise
  return base, q, opt


def engine_options(opt, **extra):
  out = dict(opt, c_log_level=1, py_log_level=1)
  out.update(extra)
  return out


def assert_same_bits(a, b):
  assert a.shape == b.shape
  assert (np.ascontiguousarray(a).view(np.uint32) == np.ascontiguousarray(b).view(np.uint32)).all()


def oracle_graph_of(engine, base, opt):
  """The engine's device-resident graph as an oracle graph over the same vectors."""
  import oracle
  levels, rows0, rows_u = engine.obj.get_graph()
  g = oracle.Graph(base, levels, opt["max_m"], opt["max_m0"], opt["dist_type"])
  g.rows0[:], g.deg0[:] = rows0, (rows0 >= 0).sum(1)
  nu = g.rowsU.shape[0]
  g.rowsU[:], g.degU[:] = rows_u[:nu], (rows_u[:nu] >= 0).sum(1)
  return g
