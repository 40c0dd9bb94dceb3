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

  value       queries/s over all ranks, queries and results resident in HBM,
              CUDA events around the search launch, max over ranks
  e2e         the same through cuhnsw_search_knn with pinned HOST buffers
              (H2D of the queries + launch + D2H of ids/distances/counts inside the timed region)
  roofline    algorithmic gather bytes of the search kernel / its event time vs the measured HBM copy peak
  parity      ids, counts and distance bits of the first query batch against the CPU restatement on
              the graph the GPU built (outside every timed region)
  value_by_ef the device-resident value at every ef of the sweep that meets the recall bar
  build_roofline  algorithmic bytes of the construction (counted by the CPU restatement on the same
              insertion schedule) / build_graph seconds vs the same peak
  cpu_baseline / --impl reference: the CPU restatement of the same build and search (oracle/) on the host cores

With N > 1 the line also carries two blocks measured after the weak-scaling steps:
  strong      ONE 10 000-query batch split N ways over the replicas (contiguous slices, results
              all-gathered to every rank), time = max over ranks including the gather; and the same
              batch through ONE cuhnsw_search_knn call on a handle whose option `devices` lists all
              N GPUs (host buffers, one host thread per GPU)
  sharded     the base-sharded mode on a reduced stand-in of the 100 M workload: N shards of 2 M x 96,
              100 000 queries on every shard, one NCCL all-gather of the per-shard rows, merge kernel

--workload runs one of the other workloads of cuhnsw_b200/datasets.py under the same protocol (the default
is the headline).  "sharded_100m" on N > 1 GPUs is the base-sharded mode at full size: rank r builds shard r
(12.5 M rows), every rank searches ALL queries of a step in its shard, the per-shard top-k rows are exchanged
with one NCCL all-gather and merged by (distance, id) on the device; value = queries answered over the union.
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
# DRAM bytes per launch of the search kernel as captured with ncu (dram__bytes_read.sum + dram__bytes_write.sum),
# keyed by workload and ef_search; the file sits beside the ncu summaries it was taken from
TRAFFIC_FILE = os.path.join(ROOT, "profiles", "search_kernel_dram_traffic.json")
DEFAULT_BATCH_MAX = 23680  # insertion batch of the engine on a 148-SM GPU: 4 x hyper_threads x SMs x 128 / block_dim
DEFAULT_RAMP_DIV = 4
# reduced stand-in of the 100 M-row sharded workload for the N > 1 line: rows per shard, queries per step
SHARD_ROWS, SHARD_QUERIES, SHARD_RECALL_QUERIES = 2_000_000, 100_000, 10_000


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
  ap.add_argument("--row-dtype", default="f32", choices=["f32", "f16", "bf16"],
                  help="storage type of the rows on the device (16-bit rows are a side measurement; distances stay fp32)")
  ap.add_argument("--ef-extra", type=int, nargs="*", default=[],
                  help="ef_search values tried after the workload's own sweep when that stops short of the recall "
                       "target (labelled as outside the sweep in the output)")
  ap.add_argument("--ef", type=int, default=None,
                  help="search at this ef_search whatever the recall sweep says (side measurements only)")
  ap.add_argument("--no-extra-blocks", action="store_true",
                  help="skip the side blocks: strong scaling and sharded search at N > 1, batches in flight at N = 1")
  ap.add_argument("--no-cpu-build", action="store_true", help="skip the CPU build (no build_roofline, no cpu build time)")
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


def captured_traffic(workload, ef, n_override, nq_override, row_dtype):
  """DRAM bytes of one search-kernel launch from the committed ncu capture of exactly this workload, or None."""
  if n_override is not None or nq_override is not None or row_dtype != "f32":
    return None
  try:
    with open(TRAFFIC_FILE) as f:
      return json.load(f).get(workload, {}).get(str(ef))
  except (OSError, ValueError):
    return None


def algorithmic_bytes_per_query(e, h, hu, d, max_m, max_m0, topk, elem_bytes=4):
  """Per-query gather bytes: E rows of d elements, H layer-0 adjacency rows, Hu upper rows,
  the query itself and the result row."""
  return e * elem_bytes * d + h * 4 * (1 + max_m0) + hu * 4 * (1 + max_m) + 4 * d + 8 * topk


def build_algorithmic_bytes(evals, row_bytes, d, elem_bytes=4):
  """Construction: one row of d elements per distance evaluation (descent, beam search, neighbour selection
  with its early exit) plus the adjacency rows read or written (ids + stored distances + degree)."""
  return evals * elem_bytes * d + row_bytes


def pick_ef(recalls):
  for ef in sorted(recalls):
    if recalls[ef] >= RECALL_TARGET:
      return ef
  return max(recalls)


def spread(ms_list):
  a = np.asarray(ms_list, np.float64)
  return {"min": float(a.min()), "median": float(np.median(a)), "max": float(a.max())}


def workload_config(workload, n, d, nq, topk, ef, recalls, opt, nr, row_dtype, sweep):
  """The `config` object; both arms print the same keys so that their lines can be compared."""
  return {"workload": workload, "n": int(n), "d": int(d), "queries_per_step_per_gpu": int(nq), "topk": int(topk),
          "ef_search": int(ef), "recall_at_10": recalls[ef], "recall_sweep": {str(k): v for k, v in recalls.items()},
          "ef_outside_sweep": [int(e) for e in recalls if e not in sweep],
          "max_m": opt["max_m"], "max_m0": opt["max_m0"], "ef_construction": opt["ef_construction"],
          "recall_queries": int(nr), "row_dtype": row_dtype}


def stored_rows(base, row_dtype):
  """The values the device holds (what the CPU arm must search to be comparable)."""
  if row_dtype == "f16":
    return base.astype(np.float16).astype(np.float32)
  if row_dtype == "bf16":
    import torch
    return torch.from_numpy(base).to(torch.bfloat16).to(torch.float32).numpy()
  return base


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


def native_oracle():
  import oracle
  try:
    oracle.build(native=True)
    return True
  except Exception:  # pylint: disable=broad-except
    return False


def truth_device():
  try:
    import torch
    return "cuda" if torch.cuda.is_available() else "cpu"
  except Exception:  # pylint: disable=broad-except
    return "cpu"


def sweep_until_target(search_ids, truth, sweep, extra):
  """recall at every ef of the sweep; when the sweep ends below the target, the extra values in turn."""
  from cuhnsw_b200 import datasets as ds
  recalls = {}
  for ef in sweep:
    recalls[ef] = ds.recall(search_ids(ef), truth)
  for ef in extra:
    if max(recalls.values()) >= RECALL_TARGET:
      break
    if ef not in recalls:
      recalls[ef] = ds.recall(search_ids(ef), truth)
  return recalls


def run_reference(args, rank, world):
  """CPU arm: the oracle port of build and search (the reference names hnswlib as its CPU
  counterpart; neither hnswlib nor a CPU path of the reference itself exists offline).  Same
  workload, same recall sample, same queries per step and the same `config` keys as the GPU arm."""
  if rank != 0:
    return
  import oracle
  from cuhnsw_b200 import datasets as ds
  n_arg, nq_arg = args.n, args.nq
  if args.workload == "sharded_100m" and n_arg is None:
    n_arg, nq_arg = 1_000_000, nq_arg or 10_000  # a 12.5 M CPU build takes minutes: 1 M sub-sample of one shard
  base, queries, spec = ds.make(args.workload, n=n_arg, nq=nq_arg)
  base = stored_rows(base, args.row_dtype)
  opt, topk = spec["opt"], spec["topk"]
  n, d = base.shape
  nq = len(queries)
  threads = host_threads()
  native = native_oracle()
  levels = ds.random_levels(n, opt["seed"], opt["level_mult"])
  t0 = time.perf_counter()
  g = oracle.build_graph(base, levels, opt["max_m"], opt["max_m0"], opt["dist_type"], opt["ef_construction"],
                         0.25, False, bmax=DEFAULT_BATCH_MAX, ramp_div=DEFAULT_RAMP_DIV, nthreads=threads, native=native)
  build_s = time.perf_counter() - t0
  nr = min(nq, args.recall_queries)
  # exact answer computed the way the GPU arm computes it (same matmul, same device when one is present), so
  # that both arms score their recall against the very same truth
  truth = ds.ground_truth(base, queries[:nr], topk, opt["dist_type"], device=truth_device())
  recalls = sweep_until_target(lambda ef: oracle.search(g, queries[:nr], topk, ef, nthreads=threads, native=native)[0],
                               truth, spec["ef_sweep"], args.ef_extra)
  ef = pick_ef(recalls)
  if args.ef is not None:
    ef = args.ef
    if ef not in recalls:
      recalls[ef] = ds.recall(oracle.search(g, queries[:nr], topk, ef, nthreads=threads, native=native)[0], truth)
  # distinct batches per step, like the GPU arm; batch 0 is the recall batch
  total = args.warmup + args.steps
  distinct = min(total, 8)
  made = [queries if s == 0 else ds.make_queries(args.workload, nq, 1 + s) for s in range(distinct)]
  for s in range(args.warmup):
    oracle.search(g, made[s % distinct], topk, ef, nthreads=threads, native=native)
  per_step = []
  for s in range(args.steps):
    t0 = time.perf_counter()
    oracle.search(g, made[(args.warmup + s) % distinct], topk, ef, nthreads=threads, native=native)
    per_step.append((time.perf_counter() - t0) * 1e3)
  el = sum(per_step) * 1e-3
  qps = args.steps * nq / el
  sample_txt = f"{args.steps} steps x {nq} queries of the workload, ef_search={ef}, {threads} threads"
  line = {
    "impl": "reference", "metric": "batch-search QPS at recall@10>=0.95", "value": qps, "unit": "queries/s",
    "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": el / args.steps * 1e3,
    "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
    "config": workload_config(args.workload, n, d, nq, topk, ef, recalls, opt, nr, args.row_dtype, spec["ef_sweep"]),
    "step_ms": spread(per_step),
    "cpu_baseline": {"value": qps, "unit": "queries/s", "cores": threads, "kind": "port", "sample": sample_txt},
    "e2e": {"value": qps, "unit": "queries/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    "build_sec_per_1M": build_s / (n / 1e6), "build_seconds": build_s, "gpu_launches": 0,
    "what": "CPU restatement of the reference's build and search (oracle/), all host threads; the reference has no "
            "CPU path of its own and hnswlib is not installed",
  }
  ref_gpu = reference_gpu_search(args, g, queries[:nr], truth, topk, opt)
  if ref_gpu is not None:
    line["reference_gpu"] = ref_gpu
  print(json.dumps(line), flush=True)


def reference_gpu_search(args, g, queries, truth, topk, opt):
  """Same-box GPU anchor: the reference's OWN kernels (its unmodified sources compiled into
  oracle/_ref/libcuhnsw_ref.so) load the index file of this workload and answer the same queries through
  their SearchGraph.  Runs in a child process (oracle/ref_gpu_search.py) so that a failure there cannot take
  the CPU arm down; only for the headline workload, only when the library and a GPU are present."""
  lib_path = os.path.join(ROOT, "oracle", "_ref", "libcuhnsw_ref.so")
  if args.workload != HEADLINE or args.n is not None or not os.path.exists(lib_path):
    return None
  import tempfile
  from oracle import index_file
  try:
    with tempfile.TemporaryDirectory() as tmp:
      index_file.save(os.path.join(tmp, "w.index"), g, opt["level_mult"], opt["ef_construction"])
      np.save(os.path.join(tmp, "queries.npy"), np.ascontiguousarray(queries, np.float32))
      np.save(os.path.join(tmp, "truth.npy"), truth)
      with open(os.path.join(tmp, "opt.json"), "w") as f:
        json.dump({"c_log_level": 1, "dist_type": opt["dist_type"], "max_m": opt["max_m"], "max_m0": opt["max_m0"],
                   "ef_construction": opt["ef_construction"], "hyper_threads": 10.0, "block_dim": 32,
                   "visited_table_size": 0, "visited_list_size": 8192, "heuristic_coef": 0.25, "seed": 777,
                   "level_mult": opt["level_mult"], "save_remains": False, "reverse_cand": False, "nrz": False,
                   "batch_size": 0}, f)
      child = subprocess.run([sys.executable, os.path.join(ROOT, "oracle", "ref_gpu_search.py"), lib_path, tmp,
                              str(topk), "200", "300"], capture_output=True, text=True, timeout=420)
    for text in reversed(child.stdout.strip().splitlines()):
      if text.startswith("{"):
        return json.loads(text)
    return {"unavailable": f"child exited {child.returncode}: {child.stderr.strip()[-200:]}"}
  except subprocess.TimeoutExpired:
    return {"unavailable": "the reference's search did not finish within 420 s"}
  except Exception as exc:  # pylint: disable=broad-except
    return {"unavailable": f"{type(exc).__name__}: {exc}"}


def run_ours(args, rank, world, local_rank):
  import torch
  import torch.distributed as dist
  from cuhnsw_b200 import CuHNSW
  from cuhnsw_b200 import datasets as ds
  from cuhnsw_b200 import multi

  if not torch.cuda.is_available():
    raise SystemExit("bench.py needs a CUDA device: the engine has no CPU path")
  torch.cuda.set_device(local_rank)
  dev = torch.device("cuda", local_rank)
  host_group = None
  if world > 1:
    dist.init_process_group("nccl", device_id=dev)
    # barriers of this group block on the host only: ranks that wait there keep their GPU idle (an NCCL barrier
    # is a kernel that spins on the GPU until every rank has arrived)
    host_group = dist.new_group(backend="gloo")

  sharded = args.workload == "sharded_100m" and world > 1
  # sharded: rank r holds shard r (its own seed); every rank sees the same query batches
  base, queries0, spec = ds.make(args.workload, n=args.n, nq=args.nq, seed_offset=rank if sharded else 0)
  if sharded:
    queries0 = ds.make_queries(args.workload, queries0.shape[0], 0)
  opt, topk = dict(spec["opt"]), spec["topk"]
  n, d = base.shape
  nq = queries0.shape[0]
  eopt = {**opt, "nrz": False, "c_log_level": 1, "py_log_level": 1, "row_dtype": args.row_dtype}
  engine = CuHNSW(eopt)
  stored = stored_rows(base, args.row_dtype)  # what the device holds; the CPU arm searches the same values
  # untimed warm-up build of a 20 000-row slice: loads the construction kernels (CUDA loads a kernel on its
  # first launch) so that the timed build measures construction, not module loading
  warm = CuHNSW(eopt)
  warm.set_data(base[:20000])
  warm.build()
  del warm
  engine.set_data(base)
  t0 = time.perf_counter()
  engine.set_random_levels()
  levels_s = time.perf_counter() - t0
  t0 = time.perf_counter()
  engine.obj.build_graph()
  build_graph_s = time.perf_counter() - t0
  build_s = levels_s + build_graph_s  # = build() of the Python API
  engine.obj.set_stream(torch.cuda.current_stream().cuda_stream)
  sampler = ClockSampler(local_rank)
  if rank == 0:
    sampler.start()

  def barrier():
    torch.cuda.synchronize()
    if world > 1:
      dist.barrier()
    torch.cuda.synchronize()

  # ef_search: smallest value of the sweep that reaches the recall target on this index
  nr = min(nq, args.recall_queries)
  searcher = None
  if sharded:
    searcher = multi.ShardedSearcher(None, rank * n, rank, world, local_search_into=multi.engine_search_into(engine.obj))
    truth = sharded_truth(base, queries0[:nr], topk, opt["dist_type"], rank * n, world, dev)
  else:
    truth = ds.ground_truth(base, queries0[:nr], topk, opt["dist_type"], device=dev)
  kept = {}

  def search_ids(ef_):
    if sharded:
      out = searcher.search(torch.from_numpy(queries0[:nr]).to(dev), topk, ef_)
      kept[ef_] = tuple(t.cpu().numpy() for t in out)
    else:
      kept[ef_] = engine.search_knn(queries0[:nr], topk, ef_)
    return kept[ef_][0]

  recalls = sweep_until_target(search_ids, truth, spec["ef_sweep"], args.ef_extra)
  ef = pick_ef(recalls)
  if args.ef is not None:
    ef = args.ef
    if ef not in recalls:
      recalls[ef] = ds.recall(search_ids(ef), truth)

  total = args.warmup + args.steps
  # distinct query batches per step (and per rank when the index is replicated); batch 0 of rank 0 is the
  # recall batch.  Large batches (100 000 queries) cycle through four distinct ones to bound memory.
  distinct = total if nq * d * 4 * total <= (1 << 30) else 4
  made = [queries0 if (s == 0 and (rank == 0 or sharded)) else
          ds.make_queries(args.workload, nq, 1 + s + (0 if sharded else 1000 * rank)) for s in range(distinct)]
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

  def step_device(s, ef_):
    flush.zero_()  # evict the index from L2 between steps (not timed)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    if sharded:
      searcher.search(q_dev[s], topk, ef_)  # local search, all-gather, merge: all on this stream
    else:
      engine.obj.search_knn_device(q_dev[s].data_ptr(), nq, topk, ef_, ids_dev.data_ptr(), dist_dev.data_ptr(),
                                   found_dev.data_ptr())
    b.record()
    return a, b

  def step_host(s, ef_):
    flush.zero_()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    if sharded:
      out = searcher.search(q_pin[s].to(dev, non_blocking=True), topk, ef_)
      for src, dst in zip(out, (ids_pin, dist_pin, found_pin)):
        dst.copy_(src, non_blocking=True)
      torch.cuda.current_stream().synchronize()  # the caller holds the answer here
    else:
      engine.obj.search_knn(q_pin[s].numpy(), topk, ef_, ids_pin.numpy(), dist_pin.numpy(), found_pin.numpy())
    b.record()
    return a, b

  def timed(step_fn, ef_):
    """W untimed + K timed steps between two barriers; returns (sum of the K event times, max over ranks;
    this rank's per-step times)."""
    for s in range(args.warmup):
      step_fn(s, ef_)
    barrier()
    evs = [step_fn(args.warmup + s, ef_) for s in range(args.steps)]
    barrier()
    per_step = [a.elapsed_time(b) for a, b in evs]
    t = torch.tensor([sum(per_step)], dtype=torch.float64, device=dev)
    if world > 1:
      dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item()), per_step

  sampler.window_open()
  engine.obj.enable_stats(True)
  ms_dev, per_step_dev = timed(step_device, ef)
  stats = engine.obj.get_stats()
  engine.obj.enable_stats(False)
  ms_e2e, per_step_e2e = timed(step_host, ef)
  sampler.window_close()
  clocks = sampler.stop() if rank == 0 else None
  # sanity of the last timed result: sorted rows, full rows
  assert int(found_pin.min()) == min(topk, n * (world if sharded else 1)), "search returned short rows"
  assert bool((dist_pin[:, 1:] >= dist_pin[:, :-1]).all()), "rows are not ascending"

  total_q = (1 if sharded else world) * nq * args.steps  # sharded: every rank works on the same queries
  # the value at every other ef that meets the bar, same protocol (outside the headline's timed region)
  value_by_ef = {str(ef): total_q / (ms_dev * 1e-3)}
  for other in sorted(recalls):
    if other != ef and recalls[other] >= RECALL_TARGET:
      ms_other, _ = timed(step_device, other)
      value_by_ef[str(other)] = total_q / (ms_other * 1e-3)

  # The same kernel on a batch ten times the size (one launch, 21 waves of warps instead of 2): a launch cannot
  # end before its longest walk does, which alone takes about 1 ms at this ef, so the 10 000-query launch of the
  # metric sits well below the throughput the kernel reaches once that walk is amortised.  Side figure, N = 1.
  large_batch = None
  if world == 1 and not sharded and args.workload == HEADLINE and args.n is None and args.nq is None:
    big = torch.from_numpy(np.concatenate([ds.make_queries(args.workload, nq, 500 + s) for s in range(10)])).to(dev)
    big_out = (torch.empty((10 * nq, topk), dtype=torch.int32, device=dev),
               torch.empty((10 * nq, topk), dtype=torch.float32, device=dev),
               torch.empty((10 * nq,), dtype=torch.int32, device=dev))
    times = []
    for s in range(6):
      flush.zero_()
      a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
      a.record()
      engine.obj.search_knn_device(big.data_ptr(), 10 * nq, topk, ef, *[t.data_ptr() for t in big_out])
      b.record()
      torch.cuda.synchronize()
      if s >= 2:
        times.append(a.elapsed_time(b))
    large_batch = {"queries_per_launch": 10 * nq, "ms_per_launch": float(np.mean(times)),
                   "value": 10 * nq / (float(np.mean(times)) * 1e-3), "unit": "queries/s"}
    del big, big_out

  # Batches in flight on several streams: the engine keeps separate scratch per stream, so the tail of one launch
  # (bounded by its longest walk) fills with the next batch.  What a serving loop gets; side figure, N = 1.
  overlapped = None
  if world == 1 and not sharded and not args.no_extra_blocks:
    try:
      overlapped = overlapped_block(args, engine, q_dev, q_pin, nq, topk, ef, dev)
    except Exception as exc:  # pylint: disable=broad-except
      overlapped = {"unavailable": f"{type(exc).__name__}: {exc}"}

  # the graph the searches ran on, for the CPU legs of rank 0 (taken before the engine is released below)
  graph_for_cpu = oracle_graph_from_engine(engine, stored, spec) if (rank == 0 and not sharded) else None
  extra_blocks = {}
  if world > 1 and not sharded and not args.no_extra_blocks:
    # a failure in a side block must not cost the line its headline
    try:
      extra_blocks["strong"] = strong_block(args, engine, eopt, base, queries0, kept[ef], topk, ef, rank, world, dev,
                                            flush, barrier, host_group)
    except Exception as exc:  # pylint: disable=broad-except
      extra_blocks["strong"] = {"unavailable": f"{type(exc).__name__}: {exc}"}
    if args.workload == HEADLINE and args.n is None:
      del engine
      engine = None
      torch.cuda.empty_cache()
      try:
        extra_blocks["sharded"] = sharded_block(args, rank, world, dev, flush, barrier)
      except Exception as exc:  # pylint: disable=broad-except
        extra_blocks["sharded"] = {"unavailable": f"{type(exc).__name__}: {exc}"}

  if rank != 0:
    if world > 1:
      dist.destroy_process_group()
    return

  value = total_q / (ms_dev * 1e-3)
  e2e = total_q / (ms_e2e * 1e-3)
  peak, peak_kind = measured_peak()
  elem = 4 if args.row_dtype == "f32" else 2
  config = workload_config(args.workload, int(n) * (world if sharded else 1), d, nq, topk, ef, recalls, opt, nr,
                           args.row_dtype, spec["ef_sweep"])
  line = {
    "metric": "batch-search QPS at recall@10>=0.95", "value": value, "unit": "queries/s", "n_gpus": world,
    "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_dev / args.steps, "higher_is_better": True,
    "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
    "config": config,
    "parallelism": (f"base sharded x{world} ({n} rows per GPU), all queries on every GPU, all-gather + merge"
                    if sharded else f"replica x{world}, queries split"),
    "timing": {"l2": "flushed between steps (256 MB write)", "step_ms_device": spread(per_step_dev),
               "step_ms_e2e": spread(per_step_e2e), "per_step_of": "rank 0"},
    "index_bytes_per_gpu": int(n * ((d + 7) // 8 * 8 * elem + (opt["max_m0"] + 7) // 8 * 8 * 4)),
    "value_by_ef": value_by_ef,
    "e2e": {"value": e2e, "unit": "queries/s", "h2d_bytes_per_step": int(nq * d * 4),
            "d2h_bytes_per_step": int(nq * topk * 8 + nq * 4), "ms_per_step": ms_e2e / args.steps},
    # per step: entry kernel, the schedule's sort kernel (one CTA; batches above 10 240 queries use CUB's
    # device-wide sort instead, which is not counted), search kernel (+ merge kernel when sharded)
    "gpu_launches": args.steps * ((3 if nq <= 10240 else 2) + (1 if sharded else 0)),
    "build_sec_per_1M": build_s / (n / 1e6), "build_seconds": build_s, "build_graph_seconds": build_graph_s,
    "level_draw_seconds": levels_s,
    "build_timing": "wall time of set_random_levels() + build_graph() (= build()) after an untimed 20 000-row warm-up build",
    "clocks": clocks,
  }
  line.update(extra_blocks)
  # roofline of the search kernel (one launch per step): exact work counts of the first batch from the CPU
  # restatement at every N (distinct evaluations; the device's own counters include repeats)
  counted_q = nq * (args.steps + args.warmup)  # the counters also saw the warm-up steps
  counts = {"evals": stats["evals"] / counted_q, "expansions": stats["expansions"] / counted_q,
            "sweeps": stats["sweeps"] / counted_q, "source": "device counters (repeat evaluations included)"}
  cpu = None
  try:
    if not sharded:
      cpu, counts, parity, cpu_build = cpu_legs(args, graph_for_cpu, stored, queries0, spec, ef, kept[ef], counts,
                                                world, nr)
      line["parity"] = parity
      if cpu_build is not None:
        bb = build_algorithmic_bytes(cpu_build["evals"], cpu_build["row_bytes"], d, elem)
        line["build_roofline"] = {
          "bound": "hbm", "achieved": bb / build_graph_s / 1e9, "peak": peak, "unit": "GB/s",
          "frac": bb / build_graph_s / 1e9 / peak, "algorithmic_bytes": bb, "seconds": build_graph_s,
          "bytes_per_node": bb / n, "evals_per_node": cpu_build["evals"] / n, "rows_per_node": cpu_build["rows"] / n,
          "counts_source": "CPU restatement on the same insertion schedule (its graph equals the GPU's)",
          "graph_equal_to_cpu_build": cpu_build["graph_equal"], "peak_source": peak_kind}
        line["cpu_build_sec_per_1M"] = cpu_build["seconds"] / (n / 1e6)
  except Exception as exc:  # pylint: disable=broad-except
    cpu = {"value": None, "unit": "queries/s", "cores": 0, "kind": "port", "sample": f"failed: {exc}"}
  bq = algorithmic_bytes_per_query(counts["evals"], counts["expansions"], counts["sweeps"], d, opt["max_m"],
                                   opt["max_m0"], topk, elem)
  achieved = bq * nq / (ms_dev / args.steps * 1e-3) / 1e9
  line["roofline"] = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                      "traffic": captured_traffic(args.workload, ef, args.n, args.nq, args.row_dtype),
                      "traffic_source": "ncu capture under profiles/ (not measured in this run)",
                      "algorithmic_bytes_per_launch": bq * nq, "peak_source": peak_kind,
                      "bytes_per_query": bq, "counts": counts}
  if large_batch is not None:
    # same per-query work as the first batch to within the scatter between batches
    large_batch["roofline_frac"] = bq * large_batch["queries_per_launch"] / (large_batch["ms_per_launch"] * 1e-3) / 1e9 / peak
    large_batch["note"] = ("side figure: one launch of ten batches; the metric's 10 000-query launch is bounded by "
                           "its longest walk, not by the kernel's throughput")
    line["large_batch"] = large_batch
  if overlapped is not None:
    if "device" in overlapped:
      overlapped["device"]["roofline_frac"] = bq * nq / (overlapped["device"]["ms_per_step"] * 1e-3) / 1e9 / peak
    line["overlapped"] = overlapped
  if cpu is not None and world == 1:
    line["cpu_baseline"] = cpu
  print(json.dumps(line), flush=True)
  if world > 1:
    dist.destroy_process_group()


def overlapped_block(args, engine, q_dev, q_pin, nq, topk, ef, dev, lanes=4):
  """The timed steps once more with consecutive batches enqueued on `lanes` streams in turn: device-resident
  through cuhnsw_search_knn_device, and from page-locked host buffers through cuhnsw_search_knn_async (copy in,
  kernels, copies out, all on the batch's stream).  Event time from before the first batch to after the last."""
  import torch
  main = torch.cuda.current_stream()
  pool = [torch.cuda.Stream(device=dev) for _ in range(lanes)]
  out_dev = [(torch.empty((nq, topk), dtype=torch.int32, device=dev),
              torch.empty((nq, topk), dtype=torch.float32, device=dev),
              torch.empty((nq,), dtype=torch.int32, device=dev)) for _ in range(lanes)]
  out_pin = [(torch.empty((nq, topk), dtype=torch.int32).pin_memory(),
              torch.empty((nq, topk), dtype=torch.float32).pin_memory(),
              torch.empty((nq,), dtype=torch.int32).pin_memory()) for _ in range(lanes)]

  def run(host, streams):
    ms = 0.0
    for count in (args.warmup, args.steps):
      torch.cuda.synchronize()
      a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
      a.record(main)
      for st in streams:
        st.wait_event(a)
      for s in range(count):
        lane = s % len(streams)
        engine.obj.set_stream(streams[lane].cuda_stream)
        if host:
          engine.obj.search_knn_async(q_pin[s % len(q_pin)].data_ptr(), nq, topk, ef,
                                      *[t.data_ptr() for t in out_pin[lane]])
        else:
          engine.obj.search_knn_device(q_dev[s % len(q_dev)].data_ptr(), nq, topk, ef,
                                       *[t.data_ptr() for t in out_dev[lane]])
      for st in streams:
        done = torch.cuda.Event()
        done.record(st)
        main.wait_event(done)
      b.record(main)
      torch.cuda.synchronize()
      ms = a.elapsed_time(b)
    return ms / args.steps

  try:
    one = run(False, pool[:1])
    dev_ms = run(False, pool)
    host_ms = run(True, pool)
  finally:
    engine.obj.set_stream(main.cuda_stream)
  # the last batch of the last lane used: full, ascending rows
  last = out_pin[(args.steps - 1) % lanes]
  assert int(last[2].min()) >= 1 and bool((last[1][:, 1:] >= last[1][:, :-1]).all())
  return {
    "streams": lanes,
    "l2": "not flushed (batches run concurrently); every batch is distinct and the index is larger than L2",
    "device": {"ms_per_step": dev_ms, "value": nq / (dev_ms * 1e-3), "unit": "queries/s"},
    "e2e": {"ms_per_step": host_ms, "value": nq / (host_ms * 1e-3), "unit": "queries/s",
            "call": "cuhnsw_search_knn_async, page-locked host buffers, copies on the batch's stream"},
    "one_stream_no_flush_ms_per_step": one,
    "note": ("side figure: the headline value and e2e run one batch at a time; here the tail of a launch, which "
             "lasts as long as its longest walk, overlaps with the next batches"),
  }


def sharded_truth(shard, queries, topk, dist_type, id_offset, world, dev):
  """Exact answer over the union of the shards: exact top-k per shard, exchanged and merged like the search's."""
  import torch
  from cuhnsw_b200 import datasets as ds
  from cuhnsw_b200 import multi
  tids, tdist = ds.ground_truth(shard, queries, topk, dist_type, device=dev, with_distances=True)
  tids = torch.from_numpy(tids).to(dev) + id_offset
  return multi.device_merge(torch.stack(multi.gather_rows(tids, world)),
                            torch.stack(multi.gather_rows(torch.from_numpy(tdist).to(dev), world)),
                            topk)[0].cpu().numpy()


def strong_block(args, engine, eopt, base, queries0, single, topk, ef, rank, world, dev, flush, barrier, host_group):
  """Strong scaling of ONE batch (rank 0's first batch, which every rank can generate): (a) one process per GPU,
  contiguous query slices, results all-gathered to every rank; (b) rank 0 alone, ONE host-buffer call on a handle
  that holds a replica on each of the N GPUs."""
  import torch
  import torch.distributed as dist
  from cuhnsw_b200 import CuHNSW
  from cuhnsw_b200 import multi
  nq = len(queries0)
  qd = torch.from_numpy(queries0).to(dev)
  splitter = multi.SplitSearcher(multi.engine_search_into(engine.obj), rank, world)

  def step():
    flush.zero_()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    out = splitter.search(qd, topk, ef)
    b.record()
    return a, b, out

  for _ in range(args.warmup):
    step()
  barrier()
  evs = [step() for _ in range(args.steps)]
  barrier()
  per_step = torch.tensor([a.elapsed_time(b) for a, b, _ in evs], dtype=torch.float64, device=dev)
  dist.all_reduce(per_step, op=dist.ReduceOp.MAX)  # a step ends when its slowest rank holds the gathered result
  ms = float(per_step.sum().item())
  out = evs[-1][2]
  same = bool((out[0].cpu().numpy() == single[0]).all() and (out[2].cpu().numpy() == single[2]).all() and
              (out[1].cpu().numpy().view(np.uint32) == single[1].view(np.uint32)).all())
  block = {"queries_per_step": nq, "ef_search": ef, "value": args.steps * nq / (ms * 1e-3), "unit": "queries/s",
           "ms_per_step": ms / args.steps, "step_ms": spread(per_step.cpu().numpy()),
           "split": f"contiguous slices of {nq // world} queries, one NCCL all-gather per result array",
           "equals_single_gpu_answer": same}
  # (b) one call, all GPUs: only rank 0 works; the other ranks wait on the host with idle GPUs
  barrier()
  if rank == 0:
    try:
      many = CuHNSW({**eopt, "devices": list(range(world))})
      many.set_data(base)
      many.build()
      q_pin = torch.from_numpy(queries0).pin_memory()
      ids_pin = torch.empty((nq, topk), dtype=torch.int32).pin_memory()
      dist_pin = torch.empty((nq, topk), dtype=torch.float32).pin_memory()
      found_pin = torch.empty((nq,), dtype=torch.int32).pin_memory()
      times = []
      for s in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        many.obj.search_knn(q_pin.numpy(), topk, ef, ids_pin.numpy(), dist_pin.numpy(), found_pin.numpy())
        if s >= args.warmup:
          times.append((time.perf_counter() - t0) * 1e3)
      block["one_call"] = {
        "value": nq * len(times) / (sum(times) * 1e-3), "unit": "queries/s", "step_ms": spread(times),
        "what": f"cuhnsw_search_knn on one handle with devices = 0..{world - 1}: host buffers, one host thread and "
                "one slice per GPU; host wall time of the blocking call (the call spans all GPUs; L2 not flushed)",
        "equals_single_gpu_answer": bool((ids_pin.numpy() == single[0]).all() and
                                         (dist_pin.numpy().view(np.uint32) == single[1].view(np.uint32)).all())}
      # (c) the same handle, batches in flight: CuHNSW.search_knn_batches sends consecutive batches to consecutive
      # GPUs, three per GPU in flight, from this one thread; numpy arrays in, numpy arrays out
      try:
        from cuhnsw_b200 import datasets as ds
        pool = [queries0] + [ds.make_queries(args.workload, nq, 700 + s) for s in range(3)]
        rounds = [pool[s % len(pool)] for s in range(24 * world)]
        list(many.search_knn_batches(rounds[:4 * world], topk, ef, in_flight=3))  # streams, buffers, kernels
        t0 = time.perf_counter()
        got = list(many.search_knn_batches(rounds, topk, ef, in_flight=3))
        wall = time.perf_counter() - t0
        block["one_process_batches"] = {
          "value": nq * len(rounds) / wall, "unit": "queries/s", "ms_per_batch": wall / len(rounds) * 1e3,
          "batches": len(rounds), "in_flight_per_gpu": 3,
          "what": f"CuHNSW.search_knn_batches on one handle with devices = 0..{world - 1}, one host thread; host "
                  "wall time from the first batch handed in to the last result handed out",
          "equals_single_gpu_answer": bool((got[0][0] == single[0]).all() and
                                           (got[len(pool)][0] == single[0]).all())}
      except Exception as exc:  # pylint: disable=broad-except
        block["one_process_batches"] = {"unavailable": f"{type(exc).__name__}: {exc}"}
      del many
    except Exception as exc:  # pylint: disable=broad-except
      block["one_call"] = {"unavailable": f"{type(exc).__name__}: {exc}"}
  torch.cuda.synchronize()
  dist.barrier(group=host_group)
  return block


def sharded_block(args, rank, world, dev, flush, barrier):
  """Base-sharded search on a stand-in of the 100 M workload that fits the time of a scaling run: rank r indexes
  its own SHARD_ROWS x 96 shard, every rank searches all SHARD_QUERIES queries of a step in its shard, one
  all_gather_into_tensor exchanges the per-shard rows and the merge kernel reads them where they landed."""
  import torch
  import torch.distributed as dist
  from cuhnsw_b200 import CuHNSW
  from cuhnsw_b200 import datasets as ds
  from cuhnsw_b200 import multi
  name = "sharded_100m"
  shard, _, spec = ds.make(name, n=SHARD_ROWS, nq=1, seed_offset=rank)
  opt, topk, ef = dict(spec["opt"]), spec["topk"], spec["ef_sweep"][0]
  queries = ds.make_queries(name, SHARD_QUERIES, 0)
  eng = CuHNSW({**opt, "nrz": False, "c_log_level": 1, "py_log_level": 1})
  eng.set_data(shard)
  t0 = time.perf_counter()
  eng.build()
  build_s = time.perf_counter() - t0
  eng.obj.set_stream(torch.cuda.current_stream().cuda_stream)
  searcher = multi.ShardedSearcher(None, rank * SHARD_ROWS, rank, world,
                                   local_search_into=multi.engine_search_into(eng.obj))
  qd = torch.from_numpy(queries).to(dev)
  nr = SHARD_RECALL_QUERIES
  truth = sharded_truth(shard, queries[:nr], topk, opt["dist_type"], rank * SHARD_ROWS, world, dev)
  steps, warm = max(3, args.steps // 4), max(1, min(args.warmup, 3))

  def step(timed):
    flush.zero_()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    out = searcher.search(qd, topk, ef, timed=timed)
    b.record()
    return a, b, out, searcher.last_exchange_events

  for _ in range(warm):
    step(False)
  barrier()
  evs = [step(True) for _ in range(steps)]
  barrier()
  times = torch.tensor([[a.elapsed_time(b), x[0].elapsed_time(x[1]), x[1].elapsed_time(x[2])] for a, b, _, x in evs],
                       dtype=torch.float64, device=dev)
  dist.all_reduce(times, op=dist.ReduceOp.MAX)
  times = times.cpu().numpy()
  out = evs[-1][2]
  ids = out[0].cpu().numpy()
  # the device merge against the host merge on the very rows the collective delivered
  gathered = searcher._bufs[(SHARD_QUERIES, topk)][1].cpu().numpy()  # pylint: disable=protected-access
  offs = np.arange(world, dtype=np.int64)[:, None, None] * SHARD_ROWS
  g_ids = np.where(gathered[:, 0] >= 0, gathered[:, 0] + offs, -1).astype(np.int32)
  h_ids, h_d, h_found = multi.merge_topk_host(g_ids, gathered[:, 1].view(np.float32), topk)
  merge_ok = bool((h_ids == ids).all() and (h_found == out[2].cpu().numpy()).all() and
                  (h_d.view(np.uint32) == out[1].cpu().numpy().view(np.uint32)).all())
  ms = float(times[:, 0].sum())
  return {"workload": f"{world} shards of {SHARD_ROWS} x {shard.shape[1]} (stand-in of the 8 x 12.5 M workload), "
                      f"{SHARD_QUERIES} queries per step on every shard",
          "ef_search": ef, "value": steps * SHARD_QUERIES / (ms * 1e-3), "unit": "queries/s", "steps": steps,
          "ms_per_step": ms / steps, "step_ms": spread(times[:, 0]),
          "exchange_ms": float(np.median(times[:, 1])), "merge_ms": float(np.median(times[:, 2])),
          "exchange": f"one all_gather_into_tensor of [{world}, 2, {SHARD_QUERIES}, {topk}] int32 "
                      f"({8 * SHARD_QUERIES * topk} bytes per rank) over NCCL, then the merge kernel",
          "recall_at_10": ds.recall(ids[:nr], truth), "recall_queries": nr,
          "merged_ids_equal_host_merge": merge_ok, "build_seconds_per_shard": build_s}


def cpu_legs(args, g, base, queries, spec, ef, gpu_answer, counts, world, nr):
  """The CPU restatement on the same graph, queries and ef: exact per-query work counts and the parity check
  at every N; at N = 1 also its timed search (bounded) and its own build of the same index."""
  import oracle
  native = native_oracle()
  topk = spec["topk"]
  threads = host_threads()
  oids, odist, ofound, cnt = oracle.search(g, queries, topk, ef, counters=True, nthreads=threads, native=native)
  exact = {"evals": float(cnt[:, 0].mean()), "expansions": float(cnt[:, 1].mean()), "sweeps": float(cnt[:, 2].mean()),
           "source": "CPU restatement, distinct evaluations, first query batch",
           "device_evals_incl_repeats": counts["evals"]}
  gi, gd, gf = gpu_answer
  parity = {"queries": int(nr), "ef_search": int(ef),
            "ids_equal": bool((gi == oids[:nr]).all()), "found_equal": bool((gf == ofound[:nr]).all()),
            "dist_bits_equal": bool((np.ascontiguousarray(gd).view(np.uint32) == odist[:nr].view(np.uint32)).all()),
            "against": "CPU restatement (oracle/) on the graph the GPU built"}
  if world > 1:
    return None, exact, parity, None
  passes, t0 = 0, time.perf_counter()
  while True:
    oracle.search(g, queries, topk, ef, nthreads=threads, native=native)
    passes += 1
    el = time.perf_counter() - t0
    if el >= args.cpu_seconds or passes >= 200:
      break
  cpu = {"value": passes * len(queries) / el, "unit": "queries/s", "cores": threads, "kind": "port",
         "sample": f"{passes} passes over the first {len(queries)}-query batch, ef_search={ef}, {el:.1f} s"}
  # one thread on a slice of the batch (about a second): what a scalar caller of the restatement gets
  few = queries[:max(1, min(len(queries), int(len(queries) * 1.5 / max(el / passes * threads, 1e-9))))]
  t0 = time.perf_counter()
  oracle.search(g, few, topk, ef, nthreads=1, native=native)
  cpu["one_thread"] = {"value": len(few) / (time.perf_counter() - t0), "unit": "queries/s",
                       "sample": f"the first {len(few)} queries of that batch"}
  cpu_build = None
  if not args.no_cpu_build and len(base) <= 2_000_000:
    opt = spec["opt"]
    t0 = time.perf_counter()
    cg = oracle.build_graph(base, g.levels, opt["max_m"], opt["max_m0"], opt["dist_type"], opt["ef_construction"],
                            0.25, False, bmax=DEFAULT_BATCH_MAX, ramp_div=DEFAULT_RAMP_DIV, nthreads=threads,
                            native=native)
    cpu_build = {"seconds": time.perf_counter() - t0, "evals": int(cg.build_counters[0]),
                 "rows": int(cg.build_counters[1]), "row_bytes": int(cg.build_counters[2]),
                 "graph_equal": bool((cg.rows0 == g.rows0).all() and (cg.rowsU == g.rowsU).all())}
    cpu["build_sec_per_1M"] = cpu_build["seconds"] / (len(base) / 1e6)
  return cpu, exact, parity, cpu_build


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
