"""ctypes front end of the CPU oracle (``hnsw_oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by the tests, by the smoke check and by the
CPU-baseline leg of the benchmark.  The product package never imports it.

The graph is exchanged as flat numpy arrays, the same logical layout the
reference flattens its level graphs into before a launch
(cpp/src/cuhnsw_build.cu:35-47,226-240), but with global node ids on every
level:

  rows0[n, max_m0], deg0[n]            level-0 adjacency
  upper_base[n]                        exclusive prefix sum of ``levels``
  rowsU[sum(levels), max_m], degU[..]  rows of levels 1..levels[i] of node i,
                                       stored consecutively from upper_base[i]
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

DIST = {"dot": 0, "l2": 1}


def build(native=False, force=False):
  """Compiles the oracle.  ``native=True`` builds a second library tuned for
  the host it runs on (used only for the timed CPU baseline)."""
  name = "liboracle_native.so" if native else "liboracle.so"
  out = os.path.join(_HERE, name)
  src = os.path.join(_HERE, "hnsw_oracle.c")
  if not force and os.path.exists(out) and os.path.getmtime(out) >= os.path.getmtime(src):
    return out
  march = "-march=native" if native else "-march=x86-64-v3"
  cmd = ["gcc", "-O3", march, "-mfma", "-ffp-contract=off", "-fno-math-errno", "-fopenmp", "-fPIC",
         "-std=c11", "-shared", "-o", out, src, "-lm"]
  subprocess.check_call(cmd)
  return out


def _load(native=False):
  global _LIB
  if _LIB is not None and not native:
    return _LIB
  path = build(native=native)
  lib = ctypes.CDLL(path)
  f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
  i32p = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")
  lib.oracle_distance.restype = ctypes.c_float
  lib.oracle_distance.argtypes = [f32p, f32p, ctypes.c_int, ctypes.c_int]
  lib.oracle_search.restype = ctypes.c_int
  lib.oracle_search.argtypes = [
    ctypes.c_int64, ctypes.c_int, ctypes.c_int, f32p, ctypes.c_int, ctypes.c_int, i32p, i32p, i32p, i32p, i32p,
    ctypes.c_int, ctypes.c_int, f32p, ctypes.c_int64, ctypes.c_int, ctypes.c_int, i32p, f32p, i32p,
    ctypes.c_void_p, ctypes.c_int, ctypes.c_int]
  lib.oracle_build.restype = ctypes.c_int
  lib.oracle_build.argtypes = [
    ctypes.c_int64, ctypes.c_int, ctypes.c_int, f32p, i32p, ctypes.c_int, ctypes.c_int, ctypes.c_int,
    ctypes.c_double, ctypes.c_int, ctypes.c_int64, ctypes.c_int64, i32p, i32p, f32p, i32p, i32p, i32p, f32p,
    ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int), ctypes.c_void_p, ctypes.c_int, ctypes.c_int]
  lib.oracle_bruteforce.restype = ctypes.c_int
  lib.oracle_bruteforce.argtypes = [
    ctypes.c_int64, ctypes.c_int, ctypes.c_int, f32p, f32p, ctypes.c_int64, ctypes.c_int, i32p, f32p, ctypes.c_int]
  lib.oracle_max_threads.restype = ctypes.c_int
  if not native:
    _LIB = lib
  return lib


def max_threads():
  return int(_load().oracle_max_threads())


def distance(a, b, dist_type):
  a = np.ascontiguousarray(a, np.float32)
  b = np.ascontiguousarray(b, np.float32)
  return float(_load().oracle_distance(a, b, a.shape[0], DIST[dist_type]))


class Graph:
  """Flat HNSW graph + vectors, as exchanged with the oracle."""

  def __init__(self, vec, levels, max_m, max_m0, dist_type):
    self.vec = np.ascontiguousarray(vec, np.float32)
    self.levels = np.ascontiguousarray(levels, np.int32)
    self.n, self.d = self.vec.shape
    self.max_m, self.max_m0, self.dist_type = int(max_m), int(max_m0), dist_type
    base = np.zeros(self.n, np.int64)
    if self.n:
      base[1:] = np.cumsum(self.levels[:-1], dtype=np.int64)
    self.upper_base = base.astype(np.int32)
    tot = int(self.levels.sum()) if self.n else 0
    self.rows0 = np.full((self.n, self.max_m0), -1, np.int32)
    self.deg0 = np.zeros(self.n, np.int32)
    self.dist0 = np.zeros((self.n, self.max_m0), np.float32)
    self.rowsU = np.full((max(tot, 1), self.max_m), -1, np.int32)
    self.degU = np.zeros(max(tot, 1), np.int32)
    self.distU = np.zeros((max(tot, 1), self.max_m), np.float32)
    self.max_level = int(self.levels.max()) if self.n else 0
    self.enter_point = int(np.argmax(self.levels == self.max_level)) if self.n else 0
    self.labels = None


def build_graph(vec, levels, max_m, max_m0, dist_type, ef_construction, heuristic_coef=0.25, save_remains=False,
                bmax=1, ramp_div=4, nthreads=0, native=False, reverse_cand=False):
  """Oracle build.  ``bmax=1`` is the strictly sequential reference-semantics
  schedule; any other value mirrors the batch schedule of the CUDA build."""
  g = Graph(vec, levels, max_m, max_m0, dist_type)
  ml, ep = ctypes.c_int(0), ctypes.c_int(0)
  counters = np.zeros(3, np.int64)  # distance evaluations, adjacency rows touched, bytes of those rows
  rc = _load(native).oracle_build(
    g.n, g.d, DIST[dist_type], g.vec, g.levels, g.max_m, g.max_m0, int(ef_construction), float(heuristic_coef),
    int(bool(save_remains)), int(bmax), int(ramp_div), g.rows0, g.deg0, g.dist0, g.upper_base, g.rowsU, g.degU,
    g.distU, ctypes.byref(ml), ctypes.byref(ep), counters.ctypes.data, int(nthreads), int(bool(reverse_cand)))
  assert rc == 0
  g.max_level, g.enter_point = ml.value, ep.value
  g.build_counters = counters
  # unused slots read -1 so that flat comparisons are well defined
  for rows, deg in ((g.rows0, g.deg0), (g.rowsU, g.degU)):
    mask = np.arange(rows.shape[1])[None, :] >= deg[:, None]
    rows[mask] = -1
  return g


def search(g, queries, topk, ef, counters=False, nthreads=0, native=False, reverse_cand=False):
  q = np.ascontiguousarray(queries, np.float32)
  if q.ndim == 1:
    q = q[None, :]
  nq = q.shape[0]
  ids = np.full((nq, topk), -1, np.int32)
  dist = np.full((nq, topk), np.inf, np.float32)
  found = np.zeros(nq, np.int32)
  cnt = np.zeros((nq, 3), np.int64) if counters else None
  rc = _load(native).oracle_search(
    g.n, g.d, DIST[g.dist_type], g.vec, g.max_m, g.max_m0, g.rows0, g.deg0, g.upper_base, g.rowsU, g.degU,
    g.max_level, g.enter_point, q, nq, int(topk), int(ef), ids, dist, found,
    cnt.ctypes.data if counters else None, int(nthreads), int(bool(reverse_cand)))
  assert rc == 0
  if g.labels is not None:
    valid = ids >= 0
    ids[valid] = g.labels[ids[valid]].astype(np.int32)
  if counters:
    return ids, dist, found, cnt
  return ids, dist, found


def bruteforce(vec, queries, topk, dist_type, nthreads=0):
  vec = np.ascontiguousarray(vec, np.float32)
  q = np.ascontiguousarray(queries, np.float32)
  ids = np.zeros((q.shape[0], topk), np.int32)
  dist = np.zeros((q.shape[0], topk), np.float32)
  _load().oracle_bruteforce(vec.shape[0], vec.shape[1], DIST[dist_type], vec, q, q.shape[0], int(topk), ids, dist,
                            int(nthreads))
  return ids, dist
