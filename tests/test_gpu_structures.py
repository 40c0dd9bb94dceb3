"""The candidate list and the visited table of the walk kernels, each alone against a host model,
through the self-test entry points of the C ABI."""
import ctypes

import numpy as np
import pytest

from cuhnsw_b200 import cuhnsw_bind

pytestmark = pytest.mark.gpu

FLAG = 1 << 31


def ordered(dist):
  """Order-preserving image of float32 bits (negative zero counts as zero)."""
  u = int(np.float32(np.float32(dist) + np.float32(0.0)).view(np.uint32))
  return (~u & 0xffffffff) if u & 0x80000000 else (u | 0x80000000)


def run_list(cap, batches, expand):
  lib = cuhnsw_bind.load_library()
  dist = np.array([d for b in batches for d, _ in b], np.float32)
  ids = np.array([i for b in batches for _, i in b], np.int32)
  begin = np.cumsum([0] + [len(b) for b in batches]).astype(np.int32)
  expand = np.array(expand, np.int32)
  keys = np.zeros(cap, np.uint64)
  size, cursor = np.zeros(1, np.int32), np.zeros(1, np.int32)
  minpos = np.zeros(max(len(batches), 1), np.int32)
  rc = lib.cuhnsw_selftest_list_merge(cap, dist.ctypes.data, ids.ctypes.data, begin.ctypes.data, len(batches),
                                      expand.ctypes.data, keys.ctypes.data, size.ctypes.data, minpos.ctypes.data,
                                      cursor.ctypes.data)
  assert rc == 0
  return [int(k) for k in keys[:size[0]]], minpos[:len(batches)].tolist(), int(cursor[0])


def model_list(cap, batches, expand):
  """Insert one by one: skip a key that is listed, insert while there is room, else replace the largest
  key if the new one is smaller.  Keys order by (distance, id)."""
  keys, flagged, minpos = [], set(), []
  for batch, nexp in zip(batches, expand):
    for k in [k for k in keys if k not in flagged][:nexp]:
      flagged.add(k)
    new = []
    for d, i in batch:
      k = (ordered(d), i)
      if k in keys:
        continue
      if len(keys) < cap:
        keys.append(k)
      elif k < max(keys):
        gone = max(keys)
        keys.remove(gone)
        flagged.discard(gone)
        if gone in new:
          new.remove(gone)
        keys.append(k)
      else:
        continue
      new.append(k)
    keys.sort()
    minpos.append(min((keys.index(k) for k in new), default=cap))
  packed = [(o << 32) | (FLAG if (o, i) in flagged else 0) | i for o, i in keys]
  open_keys = [n for n, k in enumerate(keys) if k not in flagged]
  return packed, minpos, (open_keys[0] if open_keys else len(keys))


CASES = {
  "fills then evicts": (8, [[(5.0, 1), (3.0, 2), (9.0, 3)], [(1.0, 4), (7.0, 5), (2.0, 6), (8.0, 7), (6.0, 8)],
                            [(4.0, 9), (0.5, 10), (10.0, 11)], [(0.1, 12)]], [0, 1, 2, 0]),
  "ties break by id": (6, [[(1.0, 9), (1.0, 3), (1.0, 7)], [(1.0, 5), (1.0, 1), (1.0, 8), (1.0, 2)], [(1.0, 4), (1.0, 6)]],
                       [0, 0, 2]),
  "duplicates of listed keys": (10, [[(2.0, 1), (3.0, 2)], [(2.0, 1), (1.0, 5), (3.0, 2)], [(1.0, 5)]], [0, 1, 0]),
  "negative and zero distances": (5, [[(-0.0, 4), (0.0, 2), (-3.5, 8), (-1e-30, 1)], [(-7.0, 3), (2.0, 6), (-3.5, 7)]],
                                  [0, 2]),
  "capacity one": (1, [[(4.0, 1)], [(5.0, 2)], [(3.0, 3), (2.0, 4)]], [0, 0, 1]),
  "nothing fits": (4, [[(1.0, 1), (2.0, 2), (3.0, 3), (4.0, 4)], [(9.0, 5), (8.0, 6)], []], [4, 0, 0]),
}


@pytest.mark.parametrize("name", sorted(CASES))
def test_list_merge_small_cases(name):
  cap, batches, expand = CASES[name]
  assert run_list(cap, batches, expand) == model_list(cap, batches, expand)


@pytest.mark.parametrize("cap,seed,rounds,most", [(10, 1, 120, 32), (33, 2, 120, 32), (64, 3, 120, 32),
                                                  (200, 4, 120, 32), (300, 5, 120, 32), (1000, 6, 120, 32),
                                                  (3000, 7, 900, 6), (8192, 8, 700, 20)])
def test_list_merge_random_walks(cap, seed, rounds, most):
  """Batches of 0 to `most` keys drawn from a small set of distances (so that ties and re-offers are common),
  with expansions in between, as a walk produces them.  The last two cases grow lists of more than 1024 keys,
  whose insertion places are searched span by span."""
  rng = np.random.default_rng(seed)
  pool_d = rng.standard_normal(40 if cap <= 1000 else 400).astype(np.float32)
  batches, expand, offered = [], [], []
  for _ in range(rounds):
    n = int(rng.integers(0, most + 1))
    batch = {}
    while len(batch) < n:
      if offered and rng.random() < 0.2:
        d, i = offered[int(rng.integers(len(offered)))]  # offered before: listed, evicted or rejected
      else:
        d, i = float(pool_d[int(rng.integers(len(pool_d)))]), int(rng.integers(0, 1 << 20))
      batch[i] = (d, i)  # ids are unique within a batch, as in an adjacency row
    batch = list(batch.values())
    offered.extend(batch)
    batches.append(batch)
    expand.append(int(rng.integers(0, 4)))
  # a re-offered id must come with the distance it had: one id, one distance
  seen = {}
  batches = [[(seen.setdefault(i, d), i) for d, i in b] for b in batches]
  assert run_list(cap, batches, expand) == model_list(cap, batches, expand)


@pytest.mark.parametrize("entries,n", [(64, 1000), (1024, 100_000), (2048, 1_183_514), (4096, 12_500_000),
                                        (2048, 100_000_000), (64, 2_000_000_000)])
def test_visited_table_never_invents_and_keeps_the_recent(entries, n):
  lib = cuhnsw_bind.load_library()
  rng = np.random.default_rng(entries + n)
  fresh = rng.integers(0, n, 6000).astype(np.int32)
  ids = []
  for v in fresh:
    ids.append(int(v))
    r = rng.random()
    if r < 0.15:
      ids.append(int(v))                      # again at once
    elif r < 0.3 and len(ids) > 2:
      ids.append(ids[-2])                     # the one before
    elif r < 0.4:
      ids.append(ids[int(rng.integers(len(ids)))])  # any earlier one
  ids = np.array(ids, np.int32)
  seen = np.zeros(len(ids), np.int32)
  assert lib.cuhnsw_selftest_visited(entries, n, ids.ctypes.data, len(ids), seen.ctypes.data) == 0
  before = set()
  for k, (v, s) in enumerate(zip(ids.tolist(), seen.tolist())):
    if s:
      assert v in before, f"position {k}: id {v} reported as seen but never offered"
    if k >= 1 and ids[k - 1] == v:
      assert s, "an id offered twice in a row must be remembered"
    if k >= 2 and ids[k - 2] == v and not seen[k - 2]:
      assert s, "a bucket keeps the two ids it stored last"
    before.add(v)
  # and it does remember: every id was offered while the table still had room for it
  again = [s for k, (v, s) in enumerate(zip(ids.tolist(), seen.tolist())) if k >= 1 and ids[k - 1] == v]
  assert len(again) > 100 and all(again)
