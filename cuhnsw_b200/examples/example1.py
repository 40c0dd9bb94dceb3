"""Build / search walk-through in the shape of the reference's examples/example1.py.

The reference example downloads glove-50-angular.hdf5 and compares against hnswlib; both need
the network.  This version runs the same steps (build + save, load + search, recall against
ground truth, timing of a large random query batch: example1.py:144-243) on the seeded
synthetic stand-in of that file, or on a real ann-benchmarks HDF5 file when one is given and
h5py is importable.  hnswlib arms run only if hnswlib is importable.

  python -m cuhnsw_b200.examples.example1 [--workload angular_toy] [--hdf5 path] [--topk 10] [--ef-search 300]
                                          [--row-dtype f16]
"""
import argparse
import os
import tempfile
import time

import numpy as np

from cuhnsw_b200 import CuHNSW, aux
from cuhnsw_b200 import datasets as ds

LOGGER = aux.get_logger()


def load_data(args):
  if args.hdf5:
    import h5py  # optional
    with h5py.File(args.hdf5, "r") as h5f:
      data = h5f["train"][:, :].astype(np.float32)
      queries = h5f["test"][:, :].astype(np.float32)
      neighbors = h5f["neighbors"][:, :args.topk].astype(np.int32)
    opt = {"dist_type": args.dist_type, "nrz": args.dist_type == "cosine"}
    if opt["nrz"]:
      queries /= np.linalg.norm(queries, axis=1)[:, None]
    return data, queries, neighbors, opt
  data, queries, spec = ds.make(args.workload)
  opt = dict(spec["opt"])
  truth_data = data / np.linalg.norm(data, axis=1)[:, None] if opt.get("nrz") else data
  neighbors = ds.ground_truth(truth_data, queries, args.topk, opt["dist_type"], device=args.truth_device)
  return data, queries, neighbors, opt


def run_gpu_training(data, opt, index_path):
  ch0 = CuHNSW(opt)
  ch0.set_data(data)
  start = time.time()
  ch0.build()
  el0 = time.time() - start
  LOGGER.info("elapsed time to build: %.4e sec (%.3f sec per 1M vectors)", el0, el0 / (len(data) / 1e6))
  ch0.save_index(index_path)
  return el0


def run_gpu_inference(queries, neighbors, opt, index_path, topk, ef_search):
  ch0 = CuHNSW(opt)
  ch0.load_index(index_path)
  start = time.time()
  pred_nn, _, _ = ch0.search_knn(queries, topk, ef_search)
  el0 = time.time() - start
  acc = ds.recall(pred_nn, neighbors)
  LOGGER.info("elapsed for %d queries of top@%d (ef_search: %d): %.4e sec, accuracy %.4f", len(queries), topk,
              ef_search, el0, acc)
  return el0, acc


def run_gpu_inference_large(opt, index_path, topk, ef_search, num_queries, num_dims):
  ch0 = CuHNSW(opt)
  ch0.load_index(index_path)
  queries = np.random.normal(size=(num_queries, num_dims)).astype(np.float32)
  if opt.get("nrz"):
    queries /= np.linalg.norm(queries, axis=1)[:, None]
  ch0.search_knn(queries[:1000], topk, ef_search)  # warm-up
  start = time.time()
  ch0.search_knn(queries, topk, ef_search)
  el0 = time.time() - start
  LOGGER.info("elapsed for %d random queries of top@%d (ef_search: %d): %.4e sec (%.0f queries/s)", num_queries,
              topk, ef_search, el0, num_queries / el0)
  # the same queries as a stream of 10 000-query batches, several of them in flight on the GPU
  chunks = [queries[s:s + 10000] for s in range(0, num_queries, 10000)]
  start = time.time()
  found = sum(int(cnt.sum()) for _, _, cnt in ch0.search_knn_batches(chunks, topk, ef_search))
  el1 = time.time() - start
  LOGGER.info("as %d batches in flight: %.4e sec (%.0f queries/s), %d neighbours found", len(chunks), el1,
              num_queries / el1, found)
  return el0


def run_cpu_inference(queries, neighbors, opt, index_path, topk, ef_search, num_data):
  try:
    import hnswlib
  except ImportError:
    LOGGER.info("hnswlib is not installed: CPU arm skipped")
    return None
  space = "l2" if opt["dist_type"] in ("l2", "euclidean") else "ip"
  hl0 = hnswlib.Index(space=space, dim=queries.shape[1])
  hl0.load_index(index_path, max_elements=num_data)
  hl0.set_ef(ef_search)
  start = time.time()
  labels, _ = hl0.knn_query(queries, k=topk)
  el0 = time.time() - start
  acc = ds.recall(labels.astype(np.int32), neighbors)
  LOGGER.info("hnswlib: %d queries in %.4e sec, accuracy %.4f", len(queries), el0, acc)
  return el0, acc


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("--workload", default="angular_toy", choices=sorted(ds.WORKLOADS))
  ap.add_argument("--hdf5", default=None)
  ap.add_argument("--dist-type", default="cosine")
  ap.add_argument("--topk", type=int, default=10)
  ap.add_argument("--ef-search", type=int, default=300)
  ap.add_argument("--large", type=int, default=100000, help="size of the random query batch of the timing run")
  ap.add_argument("--truth-device", default="cuda")
  ap.add_argument("--row-dtype", default="f32", choices=["f32", "f16"], help="storage type of the rows on the device")
  args = ap.parse_args()
  data, queries, neighbors, opt = load_data(args)
  opt["row_dtype"] = args.row_dtype
  with tempfile.TemporaryDirectory() as tmp:
    index_path = os.path.join(tmp, "cuhnsw.index")
    run_gpu_training(data, opt, index_path)
    run_gpu_inference(queries, neighbors, opt, index_path, args.topk, args.ef_search)
    run_cpu_inference(queries, neighbors, opt, index_path, args.topk, args.ef_search, len(data))
    run_gpu_inference_large(opt, index_path, args.topk, args.ef_search, args.large, data.shape[1])


if __name__ == "__main__":
  main()
