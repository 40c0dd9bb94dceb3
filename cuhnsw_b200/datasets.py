"""Seeded synthetic stand-ins for the benchmark files the reference measures on.

The reference's example downloads ann-benchmarks HDF5 files
(examples/example1.py:24-37: glove-50-angular, sift-128-euclidean).  Those
files are not available offline, so every workload here is a seeded mixture
of Gaussians with the shape, size and value distribution of the file it
replaces.  Nothing is read from disk.
"""
import math

import numpy as np

# name -> (n, d, n_queries, dist_type, options, search settings)
WORKLOADS = {
  # glove-50 shape, small: 100 isotropic Gaussians, L2-normalised
  "angular_toy": dict(n=100_000, d=50, nq=10_000, centres=100, sigma=0.3, seed=1001, qseed=1002, kind="angular",
                      opt=dict(dist_type="dot", nrz=True, max_m=12, max_m0=24, ef_construction=110,
                               level_mult=1.0 / math.log(24), seed=777),
                      topk=10, ef_sweep=(300,)),
  # stands in for glove-50-angular (N = 1 183 514)
  "angular_full": dict(n=1_183_514, d=50, nq=10_000, centres=1000, sigma=0.3, seed=2001, qseed=2002,
                       kind="angular",
                       opt=dict(dist_type="dot", nrz=True, max_m=12, max_m0=24, ef_construction=110,
                                level_mult=1.0 / math.log(24), seed=777),
                       topk=10, ef_sweep=(50, 100, 200, 300)),
  # stands in for sift-128-euclidean: integer-valued fp32 in 0..255
  "l2_integer": dict(n=1_000_000, d=128, nq=10_000, centres=256, sigma=40.0, seed=3001, qseed=3002, kind="integer",
                     opt=dict(dist_type="l2", max_m=16, max_m0=32, ef_construction=200,
                              level_mult=1.0 / math.log(32), seed=777),
                     topk=10, ef_sweep=(64, 128, 256)),
  # GIST-960 shape
  "highdim_l2": dict(n=1_000_000, d=960, nq=1_000, centres=500, sigma=0.05, seed=4001, qseed=4002, kind="uniform",
                     opt=dict(dist_type="l2", max_m=16, max_m0=32, ef_construction=200,
                              level_mult=1.0 / math.log(32), seed=777),
                     topk=10, ef_sweep=(100, 300, 500)),
  # one shard of the DEEP-96-shaped 100 M set (8 shards of 12.5 M, seed 5000 + shard)
  "sharded_100m": dict(n=12_500_000, d=96, nq=100_000, centres=10_000, sigma=0.3, seed=5000, qseed=5999,
                       kind="angular",
                       opt=dict(dist_type="dot", nrz=True, max_m=16, max_m0=32, ef_construction=100,
                                level_mult=1.0 / math.log(32), seed=777),
                       topk=10, ef_sweep=(128,)),
}


def _centres(kind, k, d, seed):
  rng = np.random.Generator(np.random.PCG64(seed * 7919 + 13))
  if kind == "angular":
    return rng.standard_normal((k, d), dtype=np.float32)
  if kind == "integer":
    return rng.integers(0, 96, size=(k, d)).astype(np.float32)
  return rng.random((k, d), dtype=np.float32)


def _draw(kind, centres, sigma, n, seed, chunk=262_144):
  rng = np.random.Generator(np.random.PCG64(seed))
  k, d = centres.shape
  out = np.empty((n, d), np.float32)
  for s in range(0, n, chunk):
    e = min(n, s + chunk)
    idx = rng.integers(0, k, size=e - s)
    noise = rng.standard_normal((e - s, d), dtype=np.float32)
    if kind == "integer":
      x = np.clip(np.rint(centres[idx] + np.abs(noise) * sigma), 0, 255)
    else:
      x = centres[idx] + sigma * noise
    if kind == "angular":
      x /= np.linalg.norm(x, axis=1, keepdims=True)
    out[s:e] = x
  return out


def make(name, n=None, nq=None, seed_offset=0):
  """Returns (base[n, d], queries[nq, d], spec).  ``n``/``nq`` override the
  sizes (tests use small slices of the same distribution); ``seed_offset``
  gives independent query batches or shards."""
  spec = dict(WORKLOADS[name])
  n = spec["n"] if n is None else n
  nq = spec["nq"] if nq is None else nq
  c = _centres(spec["kind"], spec["centres"], spec["d"], spec["seed"])
  base = _draw(spec["kind"], c, spec["sigma"], n, spec["seed"] + seed_offset)
  queries = _draw(spec["kind"], c, spec["sigma"], nq, spec["qseed"] + 104729 * seed_offset)
  return base, queries, spec


def make_queries(name, nq, seed_offset):
  spec = WORKLOADS[name]
  c = _centres(spec["kind"], spec["centres"], spec["d"], spec["seed"])
  return _draw(spec["kind"], c, spec["sigma"], nq, spec["qseed"] + 104729 * seed_offset)


def ground_truth(base, queries, topk, dist_type, device="cpu", chunk=None, with_distances=False):
  """Exact top-k ids by brute force (float32 matmul in chunks; ties by id).  With
  ``with_distances`` also the distances (L2: |b|^2 - 2 q.b + |q|^2), for merging shards."""
  import torch
  b = torch.as_tensor(base).to(device)
  q = torch.as_tensor(queries).to(device)
  n = b.shape[0]
  if chunk is None:
    chunk = max(1, int(2 ** 28 // max(n, 1)))
  out, out_d = [], []
  bn = (b * b).sum(1) if dist_type == "l2" else None
  for s in range(0, q.shape[0], chunk):
    qq = q[s:s + chunk]
    sc = qq @ b.T
    dist = (bn[None, :] - 2 * sc) if dist_type == "l2" else -sc
    # stable ascending sort => ties resolved towards the smaller id
    k = min(topk, n)
    vals, idx = torch.topk(dist, k, dim=1, largest=False, sorted=True)
    out.append(idx.to(torch.int32).cpu())
    if with_distances:
      out_d.append((vals + (qq * qq).sum(1, keepdim=True) if dist_type == "l2" else vals).cpu())
  if with_distances:
    return torch.cat(out).numpy(), torch.cat(out_d).numpy()
  return torch.cat(out).numpy()


def recall(pred, truth):
  """Mean of |pred ∩ truth| / k per query (examples/example1.py:166-171)."""
  k = truth.shape[1]
  hits = 0
  for p, t in zip(pred, truth):
    hits += len(set(p.tolist()) & set(t.tolist()))
  return hits / float(k * truth.shape[0])


def random_levels(n, seed, level_mult):
  """Level draw of the reference (cuhnsw/pyhnsw.py:65-71): legacy numpy
  stream seeded with ``seed``, level = int32(-ln(max(U, 1e-10)) * level_mult)."""
  rs = np.random.RandomState(seed)
  u = np.maximum(rs.uniform(size=n), 1e-10)
  return (-np.log(u) * level_mult).astype(np.int32)
