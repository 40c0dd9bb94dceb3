"""Times the reference's own GPU search on an index file (TEST / BASELINE INFRASTRUCTURE, never the product).

  python oracle/ref_gpu_search.py <libcuhnsw_ref.so> <dir> <topk> <ef> [<ef> ...]

<dir> holds w.index (hnswlib layout), opt.json (the reference's option file), queries.npy and truth.npy.
The library is the reference's unmodified sources compiled by oracle/build_ref.sh.  For every ef the
reference's LoadIndex'ed handle answers all queries through its SearchGraph (host buffers; it flattens and
uploads the graph on every call, cpp/src/cuhnsw_build.cu:226-253 of the reference), three times; the best
wall time of the call is what its example publishes (examples/example1.py:221-223).  Prints one JSON line.
"""
import ctypes
import json
import os
import sys
import time

import numpy as np


def main():
  lib_path, folder, topk = sys.argv[1], sys.argv[2], int(sys.argv[3])
  efs = [int(x) for x in sys.argv[4:]]
  lib = ctypes.CDLL(lib_path)
  lib.ref_create.restype = ctypes.c_void_p
  lib.ref_error.restype = ctypes.c_char_p
  for name in ("ref_init", "ref_load_index"):
    getattr(lib, name).argtypes = [ctypes.c_void_p, ctypes.c_char_p]
  lib.ref_search.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                             ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
  lib.ref_destroy.argtypes = [ctypes.c_void_p]
  q = np.ascontiguousarray(np.load(os.path.join(folder, "queries.npy")), np.float32)
  truth = np.load(os.path.join(folder, "truth.npy"))
  nq = len(q)
  out = {"what": "the reference's kernels (its SearchGraph: host buffers, graph flattened and uploaded on every "
                 "call) on the same index file and queries, best of 3 wall times of the call",
         "queries": int(nq), "by_ef": {}}

  def fail(why):
    print(json.dumps({"unavailable": why}), flush=True)
    sys.exit(0)

  h = lib.ref_create()
  if not h:
    fail("ref_create: " + (lib.ref_error() or b"").decode("utf8", "replace"))
  if lib.ref_init(h, os.path.join(folder, "opt.json").encode()) != 0:
    fail("ref_init: " + (lib.ref_error() or b"").decode("utf8", "replace"))
  t0 = time.perf_counter()
  if lib.ref_load_index(h, os.path.join(folder, "w.index").encode()) != 0:
    fail("ref_load_index: " + (lib.ref_error() or b"").decode("utf8", "replace"))
  out["load_index_seconds"] = time.perf_counter() - t0
  ids = np.zeros((nq, topk), np.int32)
  dist = np.zeros((nq, topk), np.float32)
  found = np.zeros(nq, np.int32)
  for ef in efs:
    best = None
    for _ in range(3):
      t0 = time.perf_counter()
      rc = lib.ref_search(h, q.ctypes.data, nq, topk, ef, ids.ctypes.data, dist.ctypes.data, found.ctypes.data)
      el = time.perf_counter() - t0
      if rc != 0:
        fail("ref_search: " + (lib.ref_error() or b"").decode("utf8", "replace"))
      best = el if best is None else min(best, el)
    hits = sum(len(set(a.tolist()) & set(b.tolist())) for a, b in zip(ids, truth))
    out["by_ef"][str(ef)] = {"seconds": best, "qps": nq / best, "recall_at_10": hits / float(truth.size)}
  lib.ref_destroy(h)
  print(json.dumps(out), flush=True)


if __name__ == "__main__":
  main()
