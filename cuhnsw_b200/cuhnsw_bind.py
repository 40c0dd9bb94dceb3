"""``CuHNSWBind``: the binding class of the reference (cuhnsw/bindings.cc:18-94),
re-expressed over the C ABI of libcuhnsw_b200.so with ctypes.

Same method names, argument meaning and error behaviour: ``init`` returns a
bool; every other failure raises ``RuntimeError`` (pybind11 turns the
reference's ``std::runtime_error`` into exactly that).  There is no CPU
fallback: if the shared library is missing, importing this module fails.
"""
import ctypes
import sys
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libcuhnsw_b200.so")

_f32p = ctypes.POINTER(ctypes.c_float)
_i32p = ctypes.POINTER(ctypes.c_int32)

# name -> (restype, argtypes); must list every symbol include/cuhnsw_b200.h declares
SIGNATURES = {
  "cuhnsw_create": (ctypes.c_void_p, []),
  "cuhnsw_destroy": (None, [ctypes.c_void_p]),
  "cuhnsw_last_error": (ctypes.c_char_p, [ctypes.c_void_p]),
  "cuhnsw_init": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_char_p]),
  "cuhnsw_set_data": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32]),
  "cuhnsw_set_random_levels": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p]),
  "cuhnsw_build_graph": (ctypes.c_int, [ctypes.c_void_p]),
  "cuhnsw_save_index": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_char_p]),
  "cuhnsw_load_index": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_char_p]),
  "cuhnsw_search_knn": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32,
                                       ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]),
  "cuhnsw_search_knn_device": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32,
                                              ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]),
  "cuhnsw_search_knn_async": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32,
                                             ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]),
  "cuhnsw_replica_count": (ctypes.c_int, [ctypes.c_void_p]),
  "cuhnsw_stream_create_on": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int32, ctypes.POINTER(ctypes.c_void_p)]),
  "cuhnsw_search_knn_async_on": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p,
                                                ctypes.c_int64, ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p,
                                                ctypes.c_void_p, ctypes.c_void_p]),
  "cuhnsw_search_knn_noalloc": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32,
                                               ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]),
  "cuhnsw_batch_distance": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64,
                                            ctypes.c_void_p]),
  "cuhnsw_set_stream": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p]),
  "cuhnsw_stream_create": (ctypes.c_int, [ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p)]),
  "cuhnsw_stream_synchronize": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p]),
  "cuhnsw_stream_destroy": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p]),
  "cuhnsw_host_alloc": (ctypes.c_void_p, [ctypes.c_void_p, ctypes.c_size_t]),
  "cuhnsw_host_free": (None, [ctypes.c_void_p, ctypes.c_void_p]),
  "cuhnsw_synchronize": (ctypes.c_int, [ctypes.c_void_p]),
  "cuhnsw_enable_stats": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int32]),
  "cuhnsw_get_stats": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p]),
  "cuhnsw_describe": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p]),
  "cuhnsw_get_graph": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]),
  "cuhnsw_last_build_seconds": (ctypes.c_double, [ctypes.c_void_p]),
  "cuhnsw_merge_topk_device": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64,
                                               ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                               ctypes.c_void_p]),
  "cuhnsw_merge_topk_gathered_device": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32,
                                                       ctypes.c_int64, ctypes.c_int32, ctypes.c_void_p,
                                                       ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]),
  "cuhnsw_selftest_list_merge": (ctypes.c_int, [ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                                ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                                ctypes.c_void_p, ctypes.c_void_p]),
  "cuhnsw_selftest_visited": (ctypes.c_int, [ctypes.c_int32, ctypes.c_int64, ctypes.c_void_p, ctypes.c_int32,
                                             ctypes.c_void_p]),
}

_lib = None


def load_library():
  global _lib
  if _lib is None:
    if not os.path.exists(LIB_PATH):
      raise ImportError(f"{LIB_PATH} is missing: build it with `make -C {os.path.join(_HERE, 'csrc')}` "
                        "(the engine has no CPU fallback)")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
      fn = getattr(lib, name)
      fn.restype = res
      fn.argtypes = args
    _lib = lib
  return _lib


IO_ERROR, PARSE_ERROR = -2, -3


class CuHNSWBind:
  def __init__(self):
    self._lib = load_library()
    self._h = self._lib.cuhnsw_create()
    if not self._h:
      raise RuntimeError("cuhnsw_create failed")
    self._num_dims = None  # row width of the index in place, asked for once per set_data / load_index
    self._stream = None
    self._pinned = {}  # address of a page-locked numpy array -> allocation

  def __del__(self):
    h, self._h = getattr(self, "_h", None), None
    if h:
      if not sys.is_finalizing():  # at interpreter exit the driver takes page-locked memory back, much faster
        for ptr in getattr(self, "_pinned", {}).values():
          self._lib.cuhnsw_host_free(h, ptr)
      self._lib.cuhnsw_destroy(h)

  def __repr__(self):
    return "<CuHNSWBind>"

  def _check(self, rc):
    if rc != 0:
      raise RuntimeError(self._lib.cuhnsw_last_error(self._h).decode("utf8", "replace"))

  # -- methods of the reference binding -------------------------------------
  def init(self, opt_path):
    if isinstance(opt_path, str):
      opt_path = opt_path.encode("utf8")
    rc = self._lib.cuhnsw_init(self._h, opt_path)
    if rc in (IO_ERROR, PARSE_ERROR):
      return False
    self._check(rc)
    return True

  def set_data(self, data):
    arr = np.ascontiguousarray(data, dtype=np.float32)
    if arr.ndim != 2:
      raise RuntimeError("data must be 2d array")
    self._num_dims = None
    self._check(self._lib.cuhnsw_set_data(self._h, arr.ctypes.data, arr.shape[0], arr.shape[1]))

  def set_random_levels(self, levels):
    arr = np.ascontiguousarray(levels, dtype=np.int32)
    if arr.ndim != 1:
      raise RuntimeError("levels must be 1d array")
    self._check(self._lib.cuhnsw_set_random_levels(self._h, arr.ctypes.data))

  def build_graph(self):
    self._check(self._lib.cuhnsw_build_graph(self._h))

  def save_index(self, fpath):
    if isinstance(fpath, str):
      fpath = fpath.encode("utf8")
    self._check(self._lib.cuhnsw_save_index(self._h, fpath))

  def load_index(self, fpath):
    if isinstance(fpath, str):
      fpath = fpath.encode("utf8")
    self._num_dims = None
    self._check(self._lib.cuhnsw_load_index(self._h, fpath))

  def _search_args(self, qdata, topk, nns, distances, found):
    """Validates what both host-buffer searches receive: the engine writes num_queries x topk items
    through the raw output pointers and reads num_queries x num_dims floats of the queries."""
    q = np.ascontiguousarray(qdata, dtype=np.float32)
    if q.ndim not in (1, 2):
      raise RuntimeError("data array must be 1d / 2d shape")
    nq = 1 if q.ndim == 1 else q.shape[0]
    if int(topk) < 1:
      raise RuntimeError("topk must be at least 1")
    if self._num_dims is None:  # fixed until the next set_data / load_index
      self._num_dims = self.describe()["num_dims"]
    num_dims = self._num_dims
    if num_dims > 0 and q.shape[-1] != num_dims:
      raise RuntimeError(f"queries have {q.shape[-1]} dimensions, the index has {num_dims}")
    for name, arr, dt in (("nns", nns, np.int32), ("distances", distances, np.float32), ("found", found, np.int32)):
      if not (isinstance(arr, np.ndarray) and arr.dtype == dt and arr.flags.c_contiguous and arr.flags.writeable):
        raise RuntimeError(f"{name} must be a writable C-contiguous {np.dtype(dt).name} array")
    if nns.size < nq * topk or distances.size < nq * topk or found.size < nq:
      raise RuntimeError("output arrays are too small")
    return q, nq

  def search_knn(self, qdata, topk, ef_search, nns, distances, found):
    q, nq = self._search_args(qdata, topk, nns, distances, found)
    self._check(self._lib.cuhnsw_search_knn(self._h, q.ctypes.data, nq, topk, ef_search, nns.ctypes.data,
                                            distances.ctypes.data, found.ctypes.data))

  # -- additions of this engine ---------------------------------------------
  def search_knn_device(self, q_ptr, nq, topk, ef_search, nns_ptr, dist_ptr, found_ptr):
    """All arguments are device addresses (ints); enqueued, not waited for."""
    self._check(self._lib.cuhnsw_search_knn_device(self._h, q_ptr, nq, topk, ef_search, nns_ptr, dist_ptr,
                                                   found_ptr))

  def search_knn_async(self, q_ptr, nq, topk, ef_search, nns_ptr, dist_ptr, found_ptr):
    """search_knn without the final wait.  All arguments are HOST addresses (ints) of page-locked buffers;
    the results are complete once the engine's stream (set_stream) has reached this point."""
    self._check(self._lib.cuhnsw_search_knn_async(self._h, q_ptr, nq, topk, ef_search, nns_ptr, dist_ptr,
                                                  found_ptr))

  def search_knn_noalloc(self, qdata, topk, ef_search, nns, distances, found):
    """search_knn for callers that cannot allocate device memory: device staging comes from a fixed
    4 MiB array inside the library (see cuhnsw_search_knn_noalloc in include/cuhnsw_b200.h)."""
    q, nq = self._search_args(qdata, topk, nns, distances, found)
    self._check(self._lib.cuhnsw_search_knn_noalloc(self._h, q.ctypes.data, nq, topk, ef_search, nns.ctypes.data,
                                                    distances.ctypes.data, found.ctypes.data))

  def batch_distance(self, src, dst):
    src = np.ascontiguousarray(src, np.int32)
    dst = np.ascontiguousarray(dst, np.int32)
    out = np.zeros(src.shape[0], np.float32)
    self._check(self._lib.cuhnsw_batch_distance(self._h, src.ctypes.data, dst.ctypes.data, src.shape[0],
                                                out.ctypes.data))
    return out

  def set_stream(self, stream_ptr):
    self._check(self._lib.cuhnsw_set_stream(self._h, stream_ptr))
    self._stream = stream_ptr

  def current_stream(self):
    """What the last set_stream was given (0 / None: the default stream)."""
    return self._stream

  def stream_create(self, replica=0):
    """A stream on the GPU of replica `replica` (0: the handle's own or first GPU)."""
    out = ctypes.c_void_p()
    self._check(self._lib.cuhnsw_stream_create_on(self._h, replica, ctypes.byref(out)))
    return out.value

  def replica_count(self):
    return int(self._lib.cuhnsw_replica_count(self._h))

  def search_knn_async_on(self, replica, stream_ptr, q_ptr, nq, topk, ef_search, nns_ptr, dist_ptr, found_ptr):
    """search_knn_async on one replica of a handle with `devices`, on a stream of that replica's GPU."""
    self._check(self._lib.cuhnsw_search_knn_async_on(self._h, replica, stream_ptr, q_ptr, nq, topk, ef_search,
                                                     nns_ptr, dist_ptr, found_ptr))

  def stream_synchronize(self, stream_ptr):
    self._check(self._lib.cuhnsw_stream_synchronize(self._h, stream_ptr))

  def stream_destroy(self, stream_ptr):
    self._check(self._lib.cuhnsw_stream_destroy(self._h, stream_ptr))
    if self._stream == stream_ptr:
      self._stream = None

  def host_array(self, shape, dtype):
    """numpy array over page-locked memory of this library; release it with host_release(array)."""
    dtype = np.dtype(dtype)
    count = int(np.prod(shape))
    nbytes = max(1, count * dtype.itemsize)
    ptr = self._lib.cuhnsw_host_alloc(self._h, nbytes)
    if not ptr:
      raise RuntimeError(f"cannot page-lock {nbytes} bytes of host memory")
    raw = (ctypes.c_char * nbytes).from_address(ptr)
    arr = np.frombuffer(raw, dtype=dtype, count=count).reshape(shape)
    self._pinned[arr.ctypes.data] = ptr
    return arr

  def host_release(self, arr):
    ptr = self._pinned.pop(arr.ctypes.data, None)
    if ptr and self._h:
      self._lib.cuhnsw_host_free(self._h, ptr)

  def synchronize(self):
    self._check(self._lib.cuhnsw_synchronize(self._h))

  def enable_stats(self, on=True):
    self._check(self._lib.cuhnsw_enable_stats(self._h, int(bool(on))))

  def get_stats(self):
    out = np.zeros(4, np.uint64)
    self._check(self._lib.cuhnsw_get_stats(self._h, out.ctypes.data))
    return dict(evals=int(out[0]), expansions=int(out[1]), sweeps=int(out[2]), inserts=int(out[3]))

  def describe(self):
    out = np.zeros(8, np.int64)
    self._check(self._lib.cuhnsw_describe(self._h, out.ctypes.data))
    keys = ("num_data", "num_dims", "max_level", "enter_point", "max_m", "max_m0", "upper_rows", "sm_count")
    return dict(zip(keys, (int(x) for x in out)))

  def get_graph(self):
    info = self.describe()
    n = info["num_data"]
    levels = np.zeros(n, np.int32)
    rows0 = np.full((n, info["max_m0"]), -1, np.int32)
    rows_u = np.full((max(info["upper_rows"], 1), info["max_m"]), -1, np.int32)
    self._check(self._lib.cuhnsw_get_graph(self._h, levels.ctypes.data, rows0.ctypes.data, rows_u.ctypes.data))
    return levels, rows0, rows_u

  def last_build_seconds(self):
    return float(self._lib.cuhnsw_last_build_seconds(self._h))
