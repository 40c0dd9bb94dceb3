"""Multi-GPU search: one process per GPU, ``torch.distributed`` for the plumbing.

The reference is single-device (its README lists multi-device support as an open task).
Two ways to use several GPUs follow from how the search partitions:

* replicated index, queries split: every rank holds the whole index and searches a
  contiguous slice of the query batch; no collective on the data path, results are the
  rank-ordered concatenation (``split_range`` + ``gather_rows``).
* base set sharded: rank r indexes rows [r*n/W, (r+1)*n/W); every rank searches ALL queries
  in its shard, local ids are offset to global ids, the per-shard top-k rows are exchanged
  with one all-gather and merged by (distance, id) (``ShardedSearcher``).

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


class ShardedSearcher:
  """Top-k over a base set sharded by contiguous id ranges.

  ``local_search(queries, topk, ef) -> (ids, dist, found)`` searches this rank's shard and
  returns LOCAL ids; ``id_offset`` is the global id of the shard's first row.  On GPUs pass
  ``device_merge`` (the C-ABI merge kernel) to keep the exchange and the merge on the device.
  """

  def __init__(self, local_search, id_offset, rank, world, group=None, device_merge=None):
    self.local_search = local_search
    self.id_offset = int(id_offset)
    self.rank, self.world, self.group = rank, world, group
    self.device_merge = device_merge

  def search(self, queries, topk, ef):
    import torch
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
    parts = gather_rows(packed, self.world, self.group)
    all_ids = torch.stack([t[0] for t in parts])
    all_d = torch.stack([t[1] for t in parts]).view(torch.float32)
    if is_tensor and self.device_merge is not None and all_ids.is_cuda:
      return self.device_merge(all_ids, all_d, topk)
    return merge_topk_host(all_ids.cpu().numpy(), all_d.cpu().numpy(), topk)


def device_merge(ids, dist, topk, stream_ptr=0):
  """ids/dist: CUDA tensors parts x nq x k.  Runs the merge kernel of the C ABI."""
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
