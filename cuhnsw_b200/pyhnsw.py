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
    self._batch_slots = []  # streams and page-locked buffers of search_knn_batches, kept between calls
    self._batches_running = False
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

  def search_knn_batches(self, batches, topk, ef_search, in_flight=4, normalize=False):
    """Generator over an iterable of query arrays: yields ``search_knn``'s triple for every batch, in order,
    while keeping up to ``in_flight`` batches on the GPU at once (on every GPU of ``devices``, in turn), each on
    a stream of its own through page-locked buffers (``cuhnsw_search_knn_async_on``).  A launch lasts as long as
    its longest walk; with the next batches in flight that tail is filled, which is worth about 1.4 x on
    10 000-query batches.  The streams and buffers stay with the index for the next call.  An addition: the
    reference searches one batch per blocking call (cuhnsw/pyhnsw.py:78-88 there)."""
    if self._batches_running:
      raise RuntimeError("search_knn_batches is already running on this index")
    obj, ef = self.obj, max(topk, ef_search)
    dims = obj.describe()["num_dims"]
    replicas = obj.replica_count()  # with the option `devices`: the batches go round the GPUs
    slots, wanted = self._batch_slots, max(1, in_flight) * replicas

    def collect(slot):
      obj.stream_synchronize(slot.stream)
      count, slot.pending = slot.pending, None
      if count == 0:
        return np.empty((0, topk), np.int32), np.empty((0, topk), np.float32), np.empty((0,), np.int32)
      return slot.nns[:count].copy(), slot.distances[:count].copy(), slot.found[:count].copy()

    self._batches_running = True
    try:
      turn = 0
      for qdata in batches:
        queries = normalize_rows(qdata) if normalize else np.asarray(qdata, dtype=np.float32)
        if queries.ndim == 1:
          queries = queries[None, :]
        count, width = queries.shape
        if width != dims:
          raise RuntimeError(f"queries have {width} dimensions, the index has {dims}")
        if len(slots) < wanted:
          replica = len(slots) % replicas
          slots.append(_BatchSlot(obj.stream_create(replica), replica))
        slot = slots[turn % min(len(slots), wanted)]
        turn += 1
        if slot.pending is not None:
          yield collect(slot)
        if count == 0:
          slot.pending = 0
          continue
        slot.fit(obj, count, width, topk)
        slot.queries[:count] = queries
        obj.search_knn_async_on(slot.replica, slot.stream, slot.queries.ctypes.data, count, topk, ef,
                                slot.nns.ctypes.data, slot.distances.ctypes.data, slot.found.ctypes.data)
        slot.pending = count
      # what is still in flight, oldest first
      used = min(len(slots), wanted)
      for k in range(used):
        slot = slots[(turn + k) % used]
        if slot.pending is not None:
          yield collect(slot)
    finally:
      for slot in slots:  # a consumer that stopped early leaves searches in flight
        if slot.pending is not None:
          obj.stream_synchronize(slot.stream)
          slot.pending = None
      self._batches_running = False


class _BatchSlot:
  """One batch in flight of ``CuHNSW.search_knn_batches``: a stream on one replica's GPU and one page-locked block
  cut into the query and result arrays."""
  __slots__ = ("stream", "replica", "capacity", "block", "queries", "nns", "distances", "found", "pending")

  def __init__(self, stream, replica):
    self.stream, self.replica = stream, replica
    self.capacity, self.block = 0, None
    self.queries = self.nns = self.distances = self.found = None
    self.pending = None  # number of queries of the batch in flight

  def fit(self, obj, count, width, topk):
    """Arrays for `count` queries of `width` dimensions and `topk` results each; grows, never shrinks."""
    if self.capacity >= count and self.queries.shape[1] == width and self.nns.shape[1] == topk:
      return
    if self.block is not None:
      obj.host_release(self.block)
    count = max(count, self.capacity)
    sizes = [count * width * 4, count * topk * 4, count * topk * 4, count * 4]
    starts = [0]
    for nbytes in sizes:  # 256-byte boundaries
      starts.append((starts[-1] + nbytes + 255) // 256 * 256)
    self.block = block = obj.host_array((starts[-1],), np.uint8)
    self.capacity = count
    self.queries = block[starts[0]:starts[0] + sizes[0]].view(np.float32).reshape(count, width)
    self.nns = block[starts[1]:starts[1] + sizes[1]].view(np.int32).reshape(count, topk)
    self.distances = block[starts[2]:starts[2] + sizes[2]].view(np.float32).reshape(count, topk)
    self.found = block[starts[3]:starts[3] + sizes[3]].view(np.int32)
