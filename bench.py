#!/usr/bin/env python
"""Benchmark of the hot path: batch kNN search (QPS at recall@10 >= 0.95) on the
"angular_full" workload (N = 1 183 514, d = 50, dot distance, max_m 12/24,
ef_construction 110, 10 000 queries per GPU per step), plus build seconds per
million vectors.  Synthetic data (seeded mixture of Gaussians with the shape of
glove-50-angular); nothing is read from disk.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One process per GPU (torchrun sets RANK/LOCAL_RANK/WORLD_SIZE).  Every rank holds
a replica of the index and searches its own query batches (weak scaling, no
data-path collective).  Rank 0 prints ONE JSON line.

--workload runs one of the other workloads of cuhnsw_b200/datasets.py under the same protocol (the default
is the headline).  "sharded_100m" on N > 1 GPUs is the base-sharded mode: rank r builds shard r (12.5 M
rows), every rank searches ALL queries of a step in its shard, the per-shard top-k rows are exchanged with
one NCCL all-gather and merged by (distance, id) on the device; value = queries answered over the union.

  value     queries/s over all ranks, queries and results resident in HBM,
            CUDA events around the search launch, max over ranks
  e2e       the same through cuhnsw_search_knn with pinned HOST buffers
            (H2D of the queries + launch + D2H of ids/distances/counts inside the timed region)
  roofline  algorithmic gather bytes of the search kernel / its event time vs the measured HBM copy peak
  cpu_baseline / --impl reference: the CPU restatement of the same search (oracle/) on the host cores
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

HEADLINE = "angular_full"
RECALL_TARGET = 0.95
FLUSH_BYTES = 256 << 20  # > 126 MB L2
# DRAM bytes of one knn_search_kernel launch of 10 000 queries, by ef_search, from the ncu captures under profiles/
NCU_TRAFFIC_BYTES = {200: 2.565e9, 300: 3.150e9}


def parse():
  ap = argparse.ArgumentParser()
  ap.add_argument("--gpus", type=int, default=1)
  ap.add_argument("--steps", type=int, default=50)
  ap.add_argument("--warmup", type=int, default=3)
  ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
  ap.add_argument("--n", type=int, default=None, help="override base size (debugging only; invalid as a bench number)")
  ap.add_argument("--nq", type=int, default=None)
  ap.add_argument("--cpu-seconds", type=float, default=12.0)
  ap.add_argument("--workload", default=HEADLINE, help="other workloads are side measurements, not the headline")
  ap.add_argument("--recall-queries", type=int, default=10000, help="queries of the first batch used for recall")
  ap.add_argument("--row-dtype", default="f32", choices=["f32", "f16"],
                  help="storage type of the rows on the device (f16 is a side measurement; distances stay fp32)")
  return ap.parse_args()


class ClockSampler:
  """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
  FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
            "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
            "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

  def __init__(self, gpu_index):
    self.gpu = gpu_index
    self.proc = None
    self.lines = []  # (arrival time, line)
    self.t0 = self.t1 = None

  def window_open(self):
    self.t0 = time.monotonic()

  def window_close(self):
    self.t1 = time.monotonic()

  def start(self):
    try:
      self.proc = subprocess.Popen(
        ["nvidia-smi", "-i", str(self.gpu), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
         "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
      self.thread = threading.Thread(target=self._read, daemon=True)
      self.thread.start()
    except OSError:
      self.proc = None

  def _read(self):
    for line in self.proc.stdout:
      self.lines.append((time.monotonic(), line.strip()))

  def stop(self):
    if self.proc is None:
      return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
    self.proc.terminate()
    try:
      self.proc.wait(timeout=5)
    except subprocess.TimeoutExpired:
      self.proc.kill()
    # nvidia-smi needs a few hundred ms to print its first sample, so it is started well before the timed
    # region; only the samples that arrived while the region ran are kept
    lines = [ln for t, ln in self.lines
             if self.t0 is not None and self.t1 is not None and self.t0 <= t <= self.t1 + 0.03]
    window = "timed region"
    if not lines:
      lines, window = [ln for _, ln in self.lines], "whole run (no sample arrived inside the timed region)"
    sm, mx, reasons = [], [], set()
    for line in lines:
      parts = [p.strip() for p in line.split(",")]
      if len(parts) < 9:
        continue
      try:
        sm.append(float(parts[1]))
        mx.append(float(parts[2]))
      except ValueError:
        continue
      for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[5:9]):
        if val.lower().startswith("active"):
          reasons.add(name)
    return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
            "samples": len(sm), "window": window, "reasons": sorted(reasons)}


def host_threads():
  """Host cores this process may use.  torchrun exports OMP_NUM_THREADS=1, which would otherwise
  throttle the CPU arm to one thread; the count is passed to the oracle explicitly."""
  try:
    return max(1, len(os.sched_getaffinity(0)))
  except AttributeError:
    return max(1, os.cpu_count() or 1)


def measured_peak():
  path = os.path.join(ROOT, "MEASURED_PEAKS.json")
  try:
    with open(path) as f:
      return float(json.load(f)["hbm_gbs"]), "measured"
  except (OSError, KeyError, ValueError):
    return 6650.0, "fallback"


def algorithmic_bytes_per_query(e, h, hu, d, max_m, max_m0, topk, elem_bytes=4):
  """Per-query gather bytes: E rows of d elements, H layer-0 adjacency rows, Hu upper rows,
  the query itself and the result row."""
  return e * elem_bytes * d + h * 4 * (1 + max_m0) + hu * 4 * (1 + max_m) + 4 * d + 8 * topk


def pick_ef(recalls):
  for ef in sorted(recalls):
    if recalls[ef] >= RECALL_TARGET:
      return ef
  return max(recalls)


def oracle_graph_from_engine(engine, base, spec):
  import oracle
  levels, rows0, rows_u = engine.obj.get_graph()
  opt = spec["opt"]
  g = oracle.Graph(base, levels, opt["max_m"], opt["max_m0"], opt["dist_type"])
  g.rows0[:] = rows0
  g.deg0[:] = (rows0 >= 0).sum(1)
  g.rowsU[:rows_u.shape[0]] = rows_u[:g.rowsU.shape[0]]
  g.degU[:] = (g.rowsU >= 0).sum(1)
  return g


def run_reference(args, rank, world):
  """CPU arm: the oracle port of the search (the reference names hnswlib as its CPU
  counterpart; neither hnswlib nor a CPU path of the reference itself exists offline)."""
  if rank != 0:
    return
  import oracle
  from cuhnsw_b200 import datasets as ds
  n_arg, nq_arg = args.n, args.nq
  if args.workload == "sharded_100m" and n_arg is None:
    n_arg, nq_arg = 1_000_000, nq_arg or 10_000  # a 12.5 M CPU build takes minutes: 1 M sub-sample of one shard
  base, queries, spec = ds.make(args.workload, n=n_arg, nq=nq_arg)
  opt, topk = spec["opt"], spec["topk"]
  n, d = base.shape
  threads = host_threads()
  try:
    oracle.build(native=True)
    native = True
  except Exception:  # pylint: disable=broad-except
    native = False
  levels = ds.random_levels(n, opt["seed"], opt["level_mult"])
  t0 = time.perf_counter()
  g = oracle.build_graph(base, levels, opt["max_m"], opt["max_m0"], opt["dist_type"], opt["ef_construction"],
                         0.25, False, bmax=23680, ramp_div=4, nthreads=threads, native=native)
  build_s = time.perf_counter() - t0
  sample = queries[:2000]
  truth = ds.ground_truth(base, sample, topk, opt["dist_type"])
  recalls = {}
  for ef in spec["ef_sweep"]:
    ids, _, _ = oracle.search(g, sample, topk, ef, nthreads=threads, native=native)
    recalls[ef] = ds.recall(ids, truth)
  ef = pick_ef(recalls)
  nq_step = min(len(queries), 5000)
  for _ in range(args.warmup):
    oracle.search(g, queries[:nq_step], topk, ef, nthreads=threads, native=native)
  t0 = time.perf_counter()
  for s in range(args.steps):
    qs = np.roll(queries, -s * 97, axis=0)[:nq_step]
    oracle.search(g, qs, topk, ef, nthreads=threads, native=native)
  el = time.perf_counter() - t0
  qps = args.steps * nq_step / el
  sample_txt = f"{args.steps} steps x {nq_step} queries of the workload, ef_search={ef}, {threads} threads"
  line = {
    "impl": "reference", "metric": "batch-search QPS at recall@10>=0.95", "value": qps, "unit": "queries/s",
    "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": el / args.steps * 1e3,
    "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
    "config": {"workload": args.workload, "n": int(n), "d": int(d), "queries_per_step": nq_step, "topk": topk,
               "ef_search": ef, "recall_at_10": recalls[ef], "recall_sweep": {str(k): v for k, v in recalls.items()},
               "max_m": opt["max_m"], "max_m0": opt["max_m0"], "ef_construction": opt["ef_construction"]},
    "cpu_baseline": {"value": qps, "unit": "queries/s", "cores": threads, "kind": "port", "sample": sample_txt},
    "e2e": {"value": qps, "unit": "queries/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    "build_sec_per_1M": build_s / (n / 1e6), "gpu_launches": 0,
  }
  print(json.dumps(line), flush=True)


def run_ours(args, rank, world, local_rank):
  import torch
  import torch.distributed as dist
  from cuhnsw_b200 import CuHNSW
  from cuhnsw_b200 import datasets as ds

  if not torch.cuda.is_available():
    raise SystemExit("bench.py needs a CUDA device: the engine has no CPU path")
  torch.cuda.set_device(local_rank)
  dev = torch.device("cuda", local_rank)
  if world > 1:
    dist.init_process_group("nccl", device_id=dev)

  sharded = args.workload == "sharded_100m" and world > 1
  # sharded: rank r holds shard r (its own seed); every rank sees the same query batches
  base, queries0, spec = ds.make(args.workload, n=args.n, nq=args.nq, seed_offset=rank if sharded else 0)
  if sharded:
    queries0 = ds.make_queries(args.workload, queries0.shape[0], 0)
  opt, topk = dict(spec["opt"]), spec["topk"]
  n, d = base.shape
  nq = queries0.shape[0]
  engine = CuHNSW({**opt, "nrz": False, "c_log_level": 1, "py_log_level": 1, "row_dtype": args.row_dtype})
  if args.row_dtype == "f16":
    stored = base.astype(np.float16).astype(np.float32)  # what the device holds; the CPU arm searches the same values
  else:
    stored = base
  # untimed warm-up build of a 20 000-row slice: loads the construction kernels (CUDA loads a kernel on its
  # first launch) so that the timed build measures construction, not module loading
  warm = CuHNSW({**opt, "nrz": False, "c_log_level": 1, "py_log_level": 1, "row_dtype": args.row_dtype})
  warm.set_data(base[:20000])
  warm.build()
  del warm
  engine.set_data(base)
  t0 = time.perf_counter()
  engine.build()
  build_s = time.perf_counter() - t0
  engine.obj.set_stream(torch.cuda.current_stream().cuda_stream)
  sampler = ClockSampler(local_rank)
  if rank == 0:
    sampler.start()

  # ef_search: smallest value of the sweep that reaches the recall target on this index
  nr = min(nq, args.recall_queries)
  searcher = None
  if sharded:
    from cuhnsw_b200 import multi
    id_offset = rank * n

    def local_search(q, k, ef_):
      out = (torch.empty((len(q), k), dtype=torch.int32, device=dev), torch.empty((len(q), k), device=dev),
             torch.empty((len(q),), dtype=torch.int32, device=dev))
      engine.obj.search_knn_device(q.data_ptr(), len(q), k, ef_, *[t.data_ptr() for t in out])
      return out

    searcher = multi.ShardedSearcher(local_search, id_offset, rank, world, device_merge=multi.device_merge)
    # exact answer over the union: exact top-k per shard, the same exchange and merge
    tids, tdist = ds.ground_truth(base, queries0[:nr], topk, opt["dist_type"], device=dev, with_distances=True)
    tids = torch.from_numpy(tids).to(dev) + id_offset
    truth = multi.device_merge(torch.stack(multi.gather_rows(tids, world)),
                               torch.stack(multi.gather_rows(torch.from_numpy(tdist).to(dev), world)),
                               topk)[0].cpu().numpy()
  else:
    truth = ds.ground_truth(base, queries0[:nr], topk, opt["dist_type"], device=dev)
  recalls = {}
  for ef in spec["ef_sweep"]:
    if sharded:
      ids = searcher.search(torch.from_numpy(queries0[:nr]).to(dev), topk, ef)[0].cpu().numpy()
    else:
      ids, _, _ = engine.search_knn(queries0[:nr], topk, ef)
    recalls[ef] = ds.recall(ids, truth)
  ef = pick_ef(recalls)

  total = args.warmup + args.steps
  # distinct query batches per step (and per rank when the index is replicated); batch 0 of rank 0 is the
  # recall batch.  Large batches (100 000 queries) cycle through four distinct ones to bound memory.
  distinct = total if nq * d * 4 * total <= (1 << 30) else 4
  made = [queries0 if (s == 0 and (rank == 0 or sharded)) else
          ds.make_queries(args.workload, nq, 1 + s + (0 if sharded else 1000 * rank)) for s in range(distinct)]
  batches = [made[s % distinct] for s in range(total)]
  q_dev_made = [torch.from_numpy(b).to(dev) for b in made]
  q_dev = [q_dev_made[s % distinct] for s in range(total)]
  ids_dev = torch.empty((nq, topk), dtype=torch.int32, device=dev)
  dist_dev = torch.empty((nq, topk), dtype=torch.float32, device=dev)
  found_dev = torch.empty((nq,), dtype=torch.int32, device=dev)
  flush = torch.empty(FLUSH_BYTES, dtype=torch.uint8, device=dev)
  q_pin_made = [torch.from_numpy(b).pin_memory() for b in made]
  q_pin = [q_pin_made[s % distinct] for s in range(total)]
  ids_pin = torch.empty((nq, topk), dtype=torch.int32).pin_memory()
  dist_pin = torch.empty((nq, topk), dtype=torch.float32).pin_memory()
  found_pin = torch.empty((nq,), dtype=torch.int32).pin_memory()

  def barrier():
    torch.cuda.synchronize()
    if world > 1:
      dist.barrier()
    torch.cuda.synchronize()

  def step_device(s):
    flush.zero_()  # evict the index from L2 between steps (not timed)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    if sharded:
      searcher.search(q_dev[s], topk, ef)  # local search, all-gather, merge: all on this stream
    else:
      engine.obj.search_knn_device(q_dev[s].data_ptr(), nq, topk, ef, ids_dev.data_ptr(), dist_dev.data_ptr(),
                                   found_dev.data_ptr())
    b.record()
    return a, b

  def step_host(s):
    flush.zero_()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    if sharded:
      out = searcher.search(q_pin[s].to(dev, non_blocking=True), topk, ef)
      for src, dst in zip(out, (ids_pin, dist_pin, found_pin)):
        dst.copy_(src, non_blocking=True)
      torch.cuda.current_stream().synchronize()  # the caller holds the answer here
    else:
      engine.obj.search_knn(q_pin[s].numpy(), topk, ef, ids_pin.numpy(), dist_pin.numpy(), found_pin.numpy())
    b.record()
    return a, b

  def timed(step_fn):
    for s in range(args.warmup):
      step_fn(s)
    barrier()
    evs = [step_fn(args.warmup + s) for s in range(args.steps)]
    barrier()
    ms = sum(a.elapsed_time(b) for a, b in evs)
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    if world > 1:
      dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())

  sampler.window_open()
  engine.obj.enable_stats(True)
  ms_dev = timed(step_device)
  stats = engine.obj.get_stats()
  engine.obj.enable_stats(False)
  ms_e2e = timed(step_host)
  sampler.window_close()
  clocks = sampler.stop() if rank == 0 else None
  # sanity of the last timed result: sorted rows, full rows
  assert int(found_pin.min()) == min(topk, n * (world if sharded else 1)), "search returned short rows"
  assert bool((dist_pin[:, 1:] >= dist_pin[:, :-1]).all()), "rows are not ascending"

  if rank != 0:
    if world > 1:
      dist.destroy_process_group()
    return

  total_q = (1 if sharded else world) * nq * args.steps  # sharded: every rank works on the same queries
  value = total_q / (ms_dev * 1e-3)
  e2e = total_q / (ms_e2e * 1e-3)
  peak, peak_kind = measured_peak()
  line = {
    "metric": "batch-search QPS at recall@10>=0.95", "value": value, "unit": "queries/s", "n_gpus": world,
    "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_dev / args.steps, "higher_is_better": True,
    "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
    "config": {"workload": args.workload, "n": int(n) * (world if sharded else 1), "d": int(d),
               "queries_per_step_per_gpu": int(nq), "topk": topk,
               "ef_search": ef, "recall_at_10": recalls[ef], "recall_sweep": {str(k): v for k, v in recalls.items()},
               "max_m": opt["max_m"], "max_m0": opt["max_m0"], "ef_construction": opt["ef_construction"],
               "parallelism": (f"base sharded x{world} ({n} rows per GPU), all queries on every GPU, all-gather + merge"
                               if sharded else f"replica x{world}, queries split"),
               "l2": "flushed between steps (256 MB write)", "recall_queries": int(nr), "row_dtype": args.row_dtype,
               "index_bytes_per_gpu": int(n * ((d + 7) // 8 * 8 * (2 if args.row_dtype == "f16" else 4) +
                                               (opt["max_m0"] + 7) // 8 * 8 * 4))},
    "e2e": {"value": e2e, "unit": "queries/s", "h2d_bytes_per_step": int(nq * d * 4),
            "d2h_bytes_per_step": int(nq * topk * 8 + nq * 4), "ms_per_step": ms_e2e / args.steps},
    "gpu_launches": args.steps * (3 if sharded else 2),  # entry kernel + search kernel (+ merge kernel when sharded); the sort between them is CUB
    "build_sec_per_1M": build_s / (n / 1e6), "build_seconds": build_s,
    "build_timing": "wall time of build() after an untimed 20 000-row warm-up build",
    "clocks": clocks,
  }
  # roofline of the search kernel (one launch per step)
  counted_q = nq * (args.steps + args.warmup)  # the counters also saw the warm-up steps
  counts = {"evals": stats["evals"] / counted_q, "expansions": stats["expansions"] / counted_q,
            "sweeps": stats["sweeps"] / counted_q, "source": "device counters (repeat evaluations included)"}
  cpu = None
  if world == 1:
    try:
      cpu, counts = cpu_baseline(engine, stored, queries0, spec, ef, args.cpu_seconds, counts)
    except Exception as exc:  # pylint: disable=broad-except
      cpu = {"value": None, "unit": "queries/s", "cores": 0, "kind": "port", "sample": f"failed: {exc}"}
  bq = algorithmic_bytes_per_query(counts["evals"], counts["expansions"], counts["sweeps"], d, opt["max_m"],
                                   opt["max_m0"], topk, 2 if args.row_dtype == "f16" else 4)
  achieved = bq * nq / (ms_dev / args.steps * 1e-3) / 1e9
  # DRAM bytes of one launch from the committed ncu capture of this exact workload (dram__bytes_read.sum +
  # dram__bytes_write.sum, profiles/knn_search_kernel_angular_full.md); null for any other shape
  traffic = NCU_TRAFFIC_BYTES.get(ef) if (args.workload == HEADLINE and args.n is None and args.nq is None and
                                          args.row_dtype == "f32") else None
  line["roofline"] = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                      "traffic": traffic, "algorithmic_bytes_per_launch": bq * nq, "peak_source": peak_kind,
                      "bytes_per_query": bq, "counts": counts}
  if cpu is not None:
    line["cpu_baseline"] = cpu
  print(json.dumps(line), flush=True)
  if world > 1:
    dist.destroy_process_group()


def cpu_baseline(engine, base, queries, spec, ef, seconds, counts):
  """Times the CPU restatement on the same index, queries and ef, all host threads, for a bounded
  number of passes; also returns the exact per-query work counts it measured."""
  import oracle
  try:
    oracle.build(native=True)
    native = True
  except Exception:  # pylint: disable=broad-except
    native = False
  g = oracle_graph_from_engine(engine, base, spec)
  topk = spec["topk"]
  threads = host_threads()
  _, _, _, cnt = oracle.search(g, queries, topk, ef, counters=True, nthreads=threads, native=native)
  exact = {"evals": float(cnt[:, 0].mean()), "expansions": float(cnt[:, 1].mean()), "sweeps": float(cnt[:, 2].mean()),
           "source": "CPU restatement, distinct evaluations, first query batch",
           "device_evals_incl_repeats": counts["evals"]}
  passes, t0 = 0, time.perf_counter()
  while True:
    oracle.search(g, queries, topk, ef, nthreads=threads, native=native)
    passes += 1
    el = time.perf_counter() - t0
    if el >= seconds or passes >= 200:
      break
  cpu = {"value": passes * len(queries) / el, "unit": "queries/s", "cores": threads, "kind": "port",
         "sample": f"{passes} passes over the first {len(queries)}-query batch, ef_search={ef}, {el:.1f} s"}
  return cpu, exact


def main():
  args = parse()
  rank = int(os.environ.get("RANK", "0"))
  world = int(os.environ.get("WORLD_SIZE", "1"))
  local_rank = int(os.environ.get("LOCAL_RANK", "0"))
  if args.impl == "reference":
    run_reference(args, rank, world)
  else:
    run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
  main()
