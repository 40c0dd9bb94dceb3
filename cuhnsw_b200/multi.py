"""Multi-GPU search: one process per GPU, ``torch.distributed`` for the plumbing.

The reference is single-device (its README lists multi-device support as an open task).
Two ways to use several GPUs follow from how the search partitions:

* replicated index, queries split: every rank holds the whole index and searches a
  contiguous slice of the query batch; no collective on the data path, results are the
  rank-ordered concatenation (``split_range`` + ``gather_rows`` / ``SplitSearcher``).
  (Inside ONE process the option ``devices`` of the engine does the same split over
  host threads; see include/cuhnsw_b200.h.)
* base set sharded: rank r indexes rows [r*n/W, (r+1)*n/W); every rank searches ALL queries
  in its shard, the per-shard top-k rows are exchanged with ONE all-gather and merged by
  (distance, id) (``ShardedSearcher``).

The collective backend is whatever the process group was created with: NCCL on GPUs,
gloo in the CPU tests (where the local search is injected).
"""
import numpy as np


def split_range(total, world, rank):
  """Contiguous, balanced slice [lo, hi) of ``total`` items for ``rank``."""
  base, rem = divmod(total, world)
  lo = rank * base + min(rank, rem)
  return lo, lo + base + (1 if rank < rem else 0)


def merge_topk_host(ids, dist, topk):
  """Reference merge on the host.  ids/dist: parts x nq x k (global ids, -1 = empty).
  Returns nq x topk rows ordered by (distance, id), and the number of valid entries."""
  parts, nq, k = ids.shape
  flat_ids = np.transpose(ids, (1, 0, 2)).reshape(nq, parts * k)
  flat_d = np.transpose(dist, (1, 0, 2)).reshape(nq, parts * k).astype(np.float32)
  flat_d = np.where(flat_ids >= 0, flat_d + np.float32(0.0), np.float32(np.inf))
  big = np.where(flat_ids >= 0, flat_ids, np.iinfo(np.int32).max)
  order = np.lexsort((big, flat_d), axis=1)[:, :topk]
  out_ids = np.take_along_axis(flat_ids, order, 1).astype(np.int32)
  out_d = np.take_along_axis(flat_d, order, 1).astype(np.float32)
  found = np.minimum((flat_ids >= 0).sum(1), topk).astype(np.int32)
  return out_ids, out_d, found


def gather_rows(local, world, group=None):
  """All-gathers equally shaped per-rank arrays/tensors; returns a list ordered by rank."""
  import torch
  import torch.distributed as dist
  t = local if isinstance(local, torch.Tensor) else torch.from_numpy(np.ascontiguousarray(local))
  if world == 1:
    return [t]
  out = [torch.empty_like(t) for _ in range(world)]
  dist.all_gather(out, t.contiguous(), group=group)
  return out


def _all_gather_into(out, local, world, group=None):
  import torch.distributed as dist
  if world == 1:
    out.view(-1).copy_(local.view(-1))
  else:
    dist.all_gather_into_tensor(out.view(-1), local.view(-1), group=group)  # flat: rank r's block lands at r * len


class SplitSearcher:
  """One query batch over a replicated index: rank r searches the contiguous slice ``split_range`` gives
  it and one all-gather puts every rank's rows at their place in the full result (the slices are padded
  to equal length for the collective).  ``search_into(q_slice, topk, ef, ids, dist, found)`` runs this
  rank's search into the given device tensors."""

  def __init__(self, search_into, rank, world, group=None):
    self.search_into, self.rank, self.world, self.group = search_into, rank, world, group
    self._bufs = {}

  def search(self, queries, topk, ef):
    import torch
    nq = queries.shape[0]
    if nq % self.world == 0:
      # equal slices: every rank's rows are gathered straight to their place in the result
      per, dev = nq // self.world, queries.device
      out_ids = torch.empty((nq, topk), dtype=torch.int32, device=dev)
      out_dist = torch.empty((nq, topk), dtype=torch.float32, device=dev)
      out_found = torch.empty((nq,), dtype=torch.int32, device=dev)
      lo = self.rank * per
      if self.world == 1:
        self.search_into(queries, topk, ef, out_ids, out_dist, out_found)
        return out_ids, out_dist, out_found
      mine = (torch.empty((per, topk), dtype=torch.int32, device=dev),
              torch.empty((per, topk), dtype=torch.float32, device=dev),
              torch.empty((per,), dtype=torch.int32, device=dev))
      self.search_into(queries[lo:lo + per], topk, ef, *mine)
      for full, part in zip((out_ids, out_dist, out_found), mine):
        _all_gather_into(full.view(self.world, -1), part.view(-1), self.world, self.group)
      return out_ids, out_dist, out_found
    per = -(-nq // self.world)  # slice length of the collective
    key = (nq, topk, queries.device)
    if key not in self._bufs:
      dev = queries.device
      # one int32 block per rank: per x topk ids, per x topk distance bits, per counts
      self._bufs[key] = (torch.empty((per * (2 * topk + 1),), dtype=torch.int32, device=dev),
                         torch.empty((self.world, per * (2 * topk + 1)), dtype=torch.int32, device=dev))
    mine, everyone = self._bufs[key]
    lo, hi = split_range(nq, self.world, self.rank)
    ids = mine[:per * topk].view(per, topk)
    dist = mine[per * topk:2 * per * topk].view(torch.float32).view(per, topk)
    found = mine[2 * per * topk:]
    if hi > lo:
      self.search_into(queries[lo:hi], topk, ef, ids[:hi - lo], dist[:hi - lo], found[:hi - lo])
    _all_gather_into(everyone, mine, self.world, self.group)
    out_ids = torch.empty((nq, topk), dtype=torch.int32, device=queries.device)
    out_dist = torch.empty((nq, topk), dtype=torch.float32, device=queries.device)
    out_found = torch.empty((nq,), dtype=torch.int32, device=queries.device)
    for r in range(self.world):
      rlo, rhi = split_range(nq, self.world, r)
      block = everyone[r]
      out_ids[rlo:rhi] = block[:per * topk].view(per, topk)[:rhi - rlo]
      out_dist[rlo:rhi] = block[per * topk:2 * per * topk].view(torch.float32).view(per, topk)[:rhi - rlo]
      out_found[rlo:rhi] = block[2 * per * topk:][:rhi - rlo]
    return out_ids, out_dist, out_found


class ShardedSearcher:
  """Top-k over a base set sharded by contiguous id ranges.

  ``id_offset`` is the global id of the shard's first row.  Two forms of the local search:

  * ``local_search(queries, topk, ef) -> (ids, dist, found)`` with LOCAL ids (numpy arrays or tensors);
    the CPU tests inject this form, and the exchange then goes through host-side packing.
  * ``local_search_into(queries, topk, ef, ids, dist, found)`` writing into given CUDA tensors: the
    search writes straight into this rank's block of the exchange buffer, one
    ``all_gather_into_tensor`` fills a ``[world, 2, nq, topk]`` int32 buffer (ids and the bit patterns of
    the distances travel together), and the merge kernel of the C ABI reads that buffer where it
    landed, adding each shard's id offset on the fly: no copy between search, collective and merge.
  """

  def __init__(self, local_search, id_offset, rank, world, group=None, device_merge=None, local_search_into=None):
    self.local_search = local_search
    self.local_search_into = local_search_into
    self.id_offset = int(id_offset)
    self.rank, self.world, self.group = rank, world, group
    self.device_merge = device_merge
    self._bufs = {}
    self._offsets = None
    self.last_exchange_events = None  # (before all-gather, after all-gather, after merge) CUDA events

  def _shard_offsets(self, device):
    import torch
    if self._offsets is None:
      mine = torch.tensor([self.id_offset], dtype=torch.int32, device=device)
      everyone = torch.empty((self.world,), dtype=torch.int32, device=device)
      _all_gather_into(everyone, mine, self.world, self.group)
      self._offsets = everyone
    return self._offsets

  def _search_on_device(self, queries, topk, ef, timed):
    import torch
    from cuhnsw_b200.cuhnsw_bind import load_library
    nq, dev = queries.shape[0], queries.device
    key = (nq, topk)
    if key not in self._bufs:
      self._bufs[key] = (torch.empty((2, nq, topk), dtype=torch.int32, device=dev),
                         torch.empty((self.world, 2, nq, topk), dtype=torch.int32, device=dev),
                         torch.empty((nq,), dtype=torch.int32, device=dev))
    mine, everyone, found_local = self._bufs[key]
    offsets = self._shard_offsets(dev)
    self.local_search_into(queries, topk, ef, mine[0], mine[1].view(torch.float32), found_local)
    stream = torch.cuda.current_stream()
    if timed:
      ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
      ev[0].record(stream)
    _all_gather_into(everyone, mine, self.world, self.group)
    if timed:
      ev[1].record(stream)
    out_ids = torch.empty((nq, topk), dtype=torch.int32, device=dev)
    out_d = torch.empty((nq, topk), dtype=torch.float32, device=dev)
    found = torch.empty((nq,), dtype=torch.int32, device=dev)
    rc = load_library().cuhnsw_merge_topk_gathered_device(
      everyone.data_ptr(), offsets.data_ptr(), self.world, nq, topk, out_ids.data_ptr(), out_d.data_ptr(),
      found.data_ptr(), stream.cuda_stream)
    if rc != 0:
      raise RuntimeError(f"cuhnsw_merge_topk_gathered_device failed ({rc})")
    if timed:
      ev[2].record(stream)
      self.last_exchange_events = ev
    return out_ids, out_d, found

  def search(self, queries, topk, ef, timed=False):
    import torch
    if self.local_search_into is not None and isinstance(queries, torch.Tensor) and queries.is_cuda:
      return self._search_on_device(queries, topk, ef, timed)
    ids, dist, _ = self.local_search(queries, topk, ef)
    is_tensor = isinstance(ids, torch.Tensor)
    if is_tensor:
      gids = torch.where(ids >= 0, ids + self.id_offset, ids)
    else:
      gids = np.where(ids >= 0, ids + self.id_offset, ids).astype(np.int32)
    # one exchange: ids and the bit patterns of the distances travel in the same int32 buffer
    gt = gids if is_tensor else torch.from_numpy(gids)
    dt = dist if is_tensor else torch.from_numpy(np.ascontiguousarray(dist, np.float32))
    packed = torch.stack([gt.to(torch.int32), dt.contiguous().view(torch.int32)])
    everyone = torch.empty((self.world,) + tuple(packed.shape), dtype=torch.int32, device=packed.device)
    _all_gather_into(everyone, packed, self.world, self.group)
    all_ids, all_d = everyone[:, 0], everyone[:, 1].view(torch.float32)
    if is_tensor and self.device_merge is not None and all_ids.is_cuda:
      return self.device_merge(all_ids, all_d, topk)
    return merge_topk_host(all_ids.cpu().numpy(), all_d.cpu().numpy(), topk)


def device_merge(ids, dist, topk, stream_ptr=0):
  """ids/dist: CUDA tensors parts x nq x k (global ids).  Runs the merge kernel of the C ABI."""
  import torch
  from cuhnsw_b200.cuhnsw_bind import load_library
  lib = load_library()
  parts, nq, k = ids.shape
  assert k == topk
  ids = ids.contiguous()
  dist = dist.contiguous()
  out_ids = torch.empty((nq, topk), dtype=torch.int32, device=ids.device)
  out_d = torch.empty((nq, topk), dtype=torch.float32, device=ids.device)
  found = torch.empty((nq,), dtype=torch.int32, device=ids.device)
  if not stream_ptr:
    stream_ptr = torch.cuda.current_stream().cuda_stream
  rc = lib.cuhnsw_merge_topk_device(ids.data_ptr(), dist.data_ptr(), parts, nq, topk, out_ids.data_ptr(),
                                    out_d.data_ptr(), found.data_ptr(), stream_ptr)
  if rc != 0:
    raise RuntimeError(f"cuhnsw_merge_topk_device failed ({rc})")
  return out_ids, out_d, found


def engine_search_into(engine_obj):
  """``local_search_into`` / ``search_into`` over a ``CuHNSWBind`` whose stream is torch's current stream."""
  def run(queries, topk, ef, ids, dist, found):
    engine_obj.search_knn_device(queries.data_ptr(), queries.shape[0], topk, ef, ids.data_ptr(), dist.data_ptr(),
                                 found.data_ptr())
  return run
