"""Multi-rank host logic on CPU: two gloo ranks, the CPU oracle as each rank's local search."""
import os
import socket
import sys

import numpy as np
import pytest

from conftest import ROOT
from cuhnsw_b200 import multi


def test_split_range_is_a_partition():
  for total in (0, 1, 7, 10, 10_000):
    for world in (1, 2, 3, 8):
      cuts = [multi.split_range(total, world, r) for r in range(world)]
      assert cuts[0][0] == 0 and cuts[-1][1] == total
      assert all(a[1] == b[0] for a, b in zip(cuts, cuts[1:]))
      assert max(hi - lo for lo, hi in cuts) - min(hi - lo for lo, hi in cuts) <= 1


def test_merge_orders_by_distance_then_id_and_handles_empty_slots():
  ids = np.array([[[4, 9, -1]], [[2, 7, 8]]], np.int32)
  dist = np.array([[[1.0, 2.0, 0.0]], [[1.0, 2.0, 3.0]]], np.float32)
  out, d, found = multi.merge_topk_host(ids, dist, 4)
  assert out.tolist() == [[2, 4, 7, 9]] and d.tolist() == [[1.0, 1.0, 2.0, 2.0]] and found.tolist() == [4]
  out, d, found = multi.merge_topk_host(ids[:1], dist[:1], 3)
  assert out.tolist() == [[4, 9, -1]] and found.tolist() == [2] and np.isinf(d[0, 2])


def _free_port():
  with socket.socket() as s:
    s.bind(("127.0.0.1", 0))
    return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
  sys.path.insert(0, ROOT)
  os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
  import torch.distributed as dist
  import oracle
  from cuhnsw_b200 import datasets as ds
  dist.init_process_group("gloo", rank=rank, world_size=world)
  base, q, spec = ds.make("angular_toy", n=4000, nq=120)
  opt = spec["opt"]
  # (a) replicated index, queries split
  levels = ds.random_levels(len(base), 777, opt["level_mult"])
  g = oracle.build_graph(base, levels, 12, 24, "dot", 60, bmax=64)
  lo, hi = multi.split_range(len(q), world, rank)
  pad = max(multi.split_range(len(q), world, r)[1] - multi.split_range(len(q), world, r)[0] for r in range(world))
  ids, _, _ = oracle.search(g, q[lo:hi], 10, 40)
  padded = np.full((pad, 10), -1, np.int32)
  padded[:hi - lo] = ids
  parts = [t.numpy() for t in multi.gather_rows(padded, world)]
  split_ids = np.concatenate([p[:multi.split_range(len(q), world, r)[1] - multi.split_range(len(q), world, r)[0]]
                              for r, p in enumerate(parts)])
  # the same through SplitSearcher (what the benchmark's strong-scaling block uses), equal and ragged slices
  import torch

  def search_into(qq, k, ef, out_ids, out_dist, out_found):
    a, b, c = oracle.search(g, qq.numpy(), k, ef)
    out_ids.copy_(torch.from_numpy(a))
    out_dist.copy_(torch.from_numpy(b))
    out_found.copy_(torch.from_numpy(c))

  splitter = multi.SplitSearcher(search_into, rank, world)
  even = splitter.search(torch.from_numpy(q), 10, 40)
  ragged = splitter.search(torch.from_numpy(q[:117]), 10, 40)
  # (b) base set sharded, all queries on every rank, all-gather + merge
  slo, shi = multi.split_range(len(base), world, rank)
  shard = base[slo:shi]
  sl = ds.random_levels(len(shard), 777, opt["level_mult"])
  sg = oracle.build_graph(shard, sl, 12, 24, "dot", 60, bmax=64)
  searcher = multi.ShardedSearcher(lambda qq, k, ef: oracle.search(sg, qq, k, ef), slo, rank, world)
  mids, md, mfound = searcher.search(q, 10, len(shard))  # ef = shard size: every shard answers exactly
  if rank == 0:
    np.savez(os.path.join(out_dir, "out.npz"), split_ids=split_ids, single_ids=oracle.search(g, q, 10, 40)[0],
             mids=mids, md=md, mfound=mfound, exact=oracle.bruteforce(base, q, 10, "dot")[0],
             even_ids=even[0].numpy(), even_dist=even[1].numpy(), even_found=even[2].numpy(),
             ragged_ids=ragged[0].numpy(), ragged_found=ragged[2].numpy(),
             single_dist=oracle.search(g, q, 10, 40)[1])
  dist.barrier()
  dist.destroy_process_group()


def test_two_ranks_query_split_and_sharded_merge(tmp_path):
  import torch.multiprocessing as mp
  port = _free_port()
  mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
  z = np.load(tmp_path / "out.npz")
  # query split over a replica = the single-process answer, row for row
  assert (z["split_ids"] == z["single_ids"]).all()
  assert (z["even_ids"] == z["single_ids"]).all() and (z["even_found"] == 10).all()
  assert (z["even_dist"].view(np.uint32) == z["single_dist"].view(np.uint32)).all()
  assert (z["ragged_ids"] == z["single_ids"][:117]).all() and (z["ragged_found"] == 10).all()
  # exact per-shard answers merged by (distance, id) = exact global answer
  assert (z["mids"] == z["exact"]).all() and (z["mfound"] == 10).all()
  assert (np.diff(z["md"], axis=1) >= 0).all()
