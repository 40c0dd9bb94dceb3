"""Golden vectors from the reference's own CUDA kernels.

Needs a GPU and oracle/_ref/libcuhnsw_ref.so (the reference's unmodified sources compiled by
oracle/build_ref.sh).  Writes into the directory given as argv[1]:

  ref_search_<case>.index   index file written by THIS repository's oracle build
  ref_search_<case>.npz     queries + what the reference's LoadIndex + SearchGraph returned on it
  ref_built_angular.index   index file the reference's own BuildGraph + SaveIndex produced
  ref_built_angular.npz     data, levels, queries and the reference's search results on its own index
  ref_quality.json          recall@10 and seconds of the reference's build on the 100 000-point workload

Run on a GPU machine:  python tests/golden/make_ref_fixtures.py <output directory>
"""
import ctypes
import json
import os
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import oracle  # noqa: E402
from oracle import index_file  # noqa: E402
from cuhnsw_b200 import datasets as ds  # noqa: E402

F32P = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
I32P = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")


class Ref:
  """The reference's host class behind oracle/ref_driver.cu."""

  def __init__(self, opt):
    self.lib = ctypes.CDLL(os.path.join(ROOT, "oracle", "_ref", "libcuhnsw_ref.so"))
    self.lib.ref_create.restype = ctypes.c_void_p
    self.lib.ref_error.restype = ctypes.c_char_p
    for name, args in (("ref_destroy", [ctypes.c_void_p]), ("ref_init", [ctypes.c_void_p, ctypes.c_char_p]),
                       ("ref_set_data", [ctypes.c_void_p, F32P, ctypes.c_int, ctypes.c_int]),
                       ("ref_set_random_levels", [ctypes.c_void_p, I32P]), ("ref_build_graph", [ctypes.c_void_p]),
                       ("ref_save_index", [ctypes.c_void_p, ctypes.c_char_p]),
                       ("ref_load_index", [ctypes.c_void_p, ctypes.c_char_p]),
                       ("ref_search", [ctypes.c_void_p, F32P, ctypes.c_int, ctypes.c_int, ctypes.c_int, I32P, F32P,
                                       I32P])):
      getattr(self.lib, name).argtypes = args
    self.h = self.lib.ref_create()
    full = dict(seed=777, c_log_level=1, py_log_level=2, max_m=12, max_m0=24, ef_construction=150, level_mult=0.0,
                save_remains=False, hyper_threads=10.0, block_dim=32, dist_type="dot", visited_table_size=0,
                visited_list_size=8192, nrz=False, reverse_cand=False, heuristic_coef=0.25)
    full.update(opt)
    with tempfile.NamedTemporaryFile("w", suffix=".json", delete=False) as f:
      json.dump(full, f)
    self.check(self.lib.ref_init(self.h, f.name.encode()))
    os.remove(f.name)

  def check(self, rc):
    if rc != 0:
      raise RuntimeError(f"reference call failed ({rc}): {self.lib.ref_error().decode()}")

  def set_data(self, data):
    self.data = np.ascontiguousarray(data, np.float32)  # the reference keeps this pointer for SaveIndex
    self.check(self.lib.ref_set_data(self.h, self.data, *self.data.shape))

  def set_levels(self, levels):
    self.check(self.lib.ref_set_random_levels(self.h, np.ascontiguousarray(levels, np.int32)))

  def build(self):
    self.check(self.lib.ref_build_graph(self.h))

  def save(self, path):
    self.check(self.lib.ref_save_index(self.h, path.encode()))

  def load(self, path):
    self.check(self.lib.ref_load_index(self.h, path.encode()))

  def search(self, q, topk, ef):
    q = np.ascontiguousarray(q, np.float32)
    nns = np.full((len(q), topk), -1, np.int32)
    dist = np.zeros((len(q), topk), np.float32)
    found = np.zeros(len(q), np.int32)
    self.check(self.lib.ref_search(self.h, q, len(q), topk, ef, nns, dist, found))
    return nns, dist, found


def small_case(name):
  if name == "angular":
    base, q, spec = ds.make("angular_toy", n=1200, nq=100)
    opt = dict(spec["opt"])
  else:  # integer-valued l2: exact distance ties
    rng = np.random.Generator(np.random.PCG64(99))
    base = rng.integers(0, 4, size=(1000, 32)).astype(np.float32)
    q = rng.integers(0, 4, size=(100, 32)).astype(np.float32)
    opt = dict(dist_type="l2", max_m=16, max_m0=32, ef_construction=100, level_mult=1 / np.log(32), seed=777)
  return base, q, opt


def main():
  out = sys.argv[1]
  os.makedirs(out, exist_ok=True)
  # (1) reference search on oracle-built indexes
  for name in ("angular", "ties"):
    base, q, opt = small_case(name)
    levels = ds.random_levels(len(base), opt["seed"], opt["level_mult"])
    g = oracle.build_graph(base, levels, opt["max_m"], opt["max_m0"], opt["dist_type"], opt["ef_construction"])
    path = os.path.join(out, f"ref_search_{name}.index")
    index_file.save(path, g, opt["level_mult"], opt["ef_construction"])
    ref = Ref({k: v for k, v in opt.items() if k != "nrz"})
    ref.load(path)
    res = {}
    for ef in (10, 40, 120):
      ids, dist, found = ref.search(q, 10, ef)
      res[f"ids_ef{ef}"], res[f"dist_ef{ef}"], res[f"found_ef{ef}"] = ids, dist, found
    np.savez_compressed(os.path.join(out, f"ref_search_{name}.npz"), queries=q, dist_type=opt["dist_type"], **res)
    print("search fixture", name, "done", flush=True)
  # (2) reference build + save on the small angular case
  base, q, opt = small_case("angular")
  levels = ds.random_levels(len(base), opt["seed"], opt["level_mult"])
  ref = Ref({k: v for k, v in opt.items() if k != "nrz"})
  ref.set_data(base)
  ref.set_levels(levels)
  ref.build()
  path = os.path.join(out, "ref_built_angular.index")
  ref.save(path)
  ref2 = Ref({k: v for k, v in opt.items() if k != "nrz"})
  ref2.load(path)
  ids, dist, found = ref2.search(q, 10, 40)
  np.savez_compressed(os.path.join(out, "ref_built_angular.npz"), levels=levels, queries=q, ids_ef40=ids,
                      dist_ef40=dist, found_ef40=found)
  print("build fixture done", flush=True)
  # (3) build quality and speed of the reference kernels on the 100 000-point workload
  base, q, spec = ds.make("angular_toy", nq=2000)
  opt = dict(spec["opt"])
  levels = ds.random_levels(len(base), opt["seed"], opt["level_mult"])
  truth = ds.ground_truth(base, q, 10, "dot")
  quality = {"workload": "angular_toy", "n": len(base), "options": {k: v for k, v in opt.items() if k != "nrz"},
             "heuristic_coef": 0.25, "hyper_threads": 10.0, "recall_at_10": {}, "search_seconds": {}}
  ref = Ref({k: v for k, v in opt.items() if k != "nrz"})
  ref.set_data(base)
  ref.set_levels(levels)
  t0 = time.perf_counter()
  ref.build()
  quality["build_seconds"] = time.perf_counter() - t0
  for ef in (20, 50, 100, 300):
    t0 = time.perf_counter()
    ids, _, _ = ref.search(q, 10, ef)
    quality["search_seconds"][str(ef)] = time.perf_counter() - t0
    quality["recall_at_10"][str(ef)] = ds.recall(ids, truth)
  with open(os.path.join(out, "ref_quality.json"), "w") as f:
    json.dump(quality, f, indent=1)
  print(json.dumps(quality), flush=True)


if __name__ == "__main__":
  main()
