"""Python front end of the engine.

API-compatible with the ``CuHNSW`` class of js1010/cuhnsw (cuhnsw/pyhnsw.py:22-88 there;
Apache-2.0, Copyright (c) 2020 Jisang Yoon): same constructor argument, same method names,
argument meaning and return values, so that a user of that package switches by changing one
import.  The implementation is this project's own: the options travel to the C ABI as a JSON
file (the binding's ``init`` takes a path, cuhnsw/bindings.cc:22-24), the vectors are handed
over once, and every search is one call into the device-resident index.
"""
import json
import os
import tempfile

import numpy as np

from cuhnsw_b200 import aux
from cuhnsw_b200.cuhnsw_bind import CuHNSWBind

# dist_type spellings the reference accepts (pyhnsw.py:19,29-31 there) and the engine's two metrics
_METRIC_OF = {"l2": "l2", "euclidean": "l2", "dot": "dot", "ip": "dot", "cosine": "dot"}
_MIN_UNIFORM = 1e-10  # floor of the uniform draw before the logarithm of the level formula
_MAX_BLOCK_DIM = 1024
_WARP = 32


def normalize_rows(x):
  """L2-normalised float32 copy of a vector or of the rows of a matrix.  The engine normalises the
  BASE rows when ``nrz`` is set but, like the reference, never the queries (its example does that by
  hand, examples/example1.py:158-159); angular workloads pass their queries through this first."""
  x = np.array(x, dtype=np.float32, copy=True)
  norm = np.linalg.norm(x, axis=-1, keepdims=True)
  np.divide(x, norm, out=x, where=norm > 0)
  return x


class CuHNSW:
  """HNSW index that lives on the GPU: ``set_data`` -> ``build`` (or ``load_index``) -> ``search_knn``."""

  def __init__(self, opt=None):
    cfg = aux.get_opt_as_proto({} if opt is None else opt)
    if cfg.dist_type not in _METRIC_OF:
      raise AssertionError(f"unknown dist_type {cfg.dist_type!r}; choose from {sorted(_METRIC_OF)}")
    # the aliases only rename the metric; "cosine" does not switch nrz on (callers set nrz themselves)
    cfg.dist_type = _METRIC_OF[cfg.dist_type]
    if not cfg.level_mult:
      cfg.level_mult = 1.0 / np.log(cfg.max_m)
    if cfg.block_dim > _MAX_BLOCK_DIM or cfg.block_dim % _WARP:
      raise AssertionError(f"invalid block dim ({cfg.block_dim}, warp size: {_WARP})")
    self.opt = cfg
    self.logger = aux.get_logger("cuhnsw", cfg.py_log_level)
    self.data = None
    self.obj = CuHNSWBind()
    text = json.dumps(aux.proto_to_dict(cfg), indent=2)
    self.logger.debug("opt: %s", text)
    fd, path = tempfile.mkstemp(suffix=".json", text=True)
    try:
      with os.fdopen(fd, "w") as out:
        out.write(text)
      if not self.obj.init(path.encode("utf8")):
        raise AssertionError(f"failed to load {path}")
    finally:
      os.remove(path)

  # -- index construction ----------------------------------------------------
  def set_data(self, data):
    rows = np.array(data, dtype=np.float32, copy=True)
    if self.opt.nrz:
      if self.opt.dist_type == "l2":
        self.logger.warning("it is not common to set nrz = True and dist_type = l2")
      rows /= np.linalg.norm(rows, axis=1, keepdims=True)
    self.data = rows
    self.logger.info("data shape: %d x %d", *rows.shape)
    self.obj.set_data(rows)

  def set_random_levels(self):
    """level(i) = int32(-ln(max(U_i, 1e-10)) * level_mult) with U from numpy's legacy generator seeded
    with ``seed``: the stream the reference draws from (pyhnsw.py:65-71 there), so that an index
    built here has the level structure the reference would give the same data."""
    stream = np.random.RandomState(self.opt.seed)
    u = stream.uniform(size=self.data.shape[0])
    np.maximum(u, _MIN_UNIFORM, out=u)
    self.obj.set_random_levels((-np.log(u) * self.opt.level_mult).astype(np.int32))

  def build(self):
    self.set_random_levels()
    self.obj.build_graph()

  # -- index file (hnswlib layout) ---------------------------------------------
  def save_index(self, fpath):
    self.obj.save_index(os.fsencode(fpath))

  def load_index(self, fpath):
    self.obj.load_index(os.fsencode(fpath))

  # -- search ----------------------------------------------------------------
  def search_knn(self, qdata, topk, ef_search, normalize=False):
    """Returns (nns int32[Q, topk], distances float32[Q, topk], found_cnt int32[Q]).  ``ef_search``
    below ``topk`` is raised to ``topk``.  ``normalize`` (an addition) L2-normalises the queries first."""
    queries = normalize_rows(qdata) if normalize else np.asarray(qdata, dtype=np.float32)
    count = 1 if queries.ndim == 1 else queries.shape[0]
    nns = np.empty((count, topk), np.int32)
    distances = np.empty((count, topk), np.float32)
    found_cnt = np.empty((count,), np.int32)
    self.obj.search_knn(queries, topk, max(topk, ef_search), nns, distances, found_cnt)
    return nns, distances, found_cnt
